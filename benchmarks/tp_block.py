"""Tensor-parallel Llama-3-8B shaped block (hidden 4096, FFN 14336, 4096 tokens per step, bf16,
random weights): fused all-gather->GEMM and GEMM->reduce-scatter kernels against the same block
made of cuBLAS GEMMs and NCCL collectives.  Device-timed, max over ranks.  The roofline of each
fused kernel is the slower of its FLOPs at the measured cuBLAS peak and its NVLink bytes at the
measured 770 GB/s per direction (900 GB/s nominal shown as well).

  python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/tp_block.py
"""
from __future__ import annotations

import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from benchmarks.sweep import _time_loop  # noqa: E402


def main():
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MINI_NCCL_BOOTSTRAP_PORT", str(int(os.environ.get("MASTER_PORT", "29500")) + 17))
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    import mini_nccl_b200 as mn
    from mini_nccl_b200.ops import gemm_status
    from mini_nccl_b200.parallel import TensorParallelAttnOut, TensorParallelMLP

    tokens, hidden, ffn = 4096, 4096, 14336
    comm = mn.Communicator(world, rank, os.environ["MASTER_ADDR"])
    peak = 1590.0
    try:
        peak = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops_sustained"]
    except Exception:
        pass
    res = {"world": world, "tokens": tokens, "hidden": hidden, "ffn": ffn}
    for n_comm in ((0,) if os.environ.get("TP_BLOCK_QUICK") else (0, 16, 36)):
        mlp = TensorParallelMLP(comm, tokens, hidden, ffn, n_comm_ctas=n_comm)
        x = (torch.randn(tokens // world, hidden, device="cuda") * 0.5).to(torch.bfloat16)
        mlp.input_shard.copy_(x)
        y = mlp.forward()
        y_ref = mlp.forward_unfused(x)
        torch.cuda.synchronize()
        err = (y.float() - y_ref.float()).abs().max().item() / (y_ref.float().abs().max().item() + 1e-9)
        ms_ag = _time_loop(lambda: mlp.ag_gemm(mlp.w_gate_up, out=mlp._h), 30, 5, world)
        ms_rs = _time_loop(lambda: mlp.gemm_rs(mlp._act, mlp.w_down), 30, 5, world)
        ms_fused = _time_loop(lambda: mlp.forward(), 30, 5, world)
        res[f"ncomm{n_comm}"] = {"ag_gemm_us": round(ms_ag * 1e3, 1), "gemm_rs_us": round(ms_rs * 1e3, 1),
                                 "mlp_fused_us": round(ms_fused * 1e3, 1), "rel_err_vs_unfused": round(err, 5),
                                 "rs_in_switch": bool(mlp.gemm_rs.in_switch), "status": gemm_status()}
        if n_comm == 0:
            ms_unf = _time_loop(lambda: mlp.forward_unfused(x), 30, 5, world)
            res["mlp_cublas_nccl_us"] = round(ms_unf * 1e3, 1)
            fl = world and 2.0 * tokens * hidden * (ffn // world)
            link = 0.770e12
            # all-gather -> GEMM: 2*M*(2F/R)*H flops; ingress (R-1)/R * M*H*2 bytes
            t_ag = max(2 * fl / (peak * 1e12), (world - 1) / world * tokens * hidden * 2 / link)
            t_rs = max(fl / (peak * 1e12), (world - 1) / world * tokens * hidden * 2 / link)
            res["roofline_us"] = {"ag_gemm": round(t_ag * 1e6, 1), "gemm_rs": round(t_rs * 1e6, 1),
                                  "peak_tflops_used": peak, "link_GBps_used": 770}
        del mlp
    att = TensorParallelAttnOut(comm, tokens, hidden)
    a = (torch.randn(tokens, hidden // world, device="cuda") * 0.5).to(torch.bfloat16)
    res["attn_out_fused_us"] = round(_time_loop(lambda: att.forward(a), 30, 5, world) * 1e3, 1)
    res["attn_out_cublas_nccl_us"] = round(_time_loop(lambda: att.forward_unfused(a), 30, 5, world) * 1e3, 1)
    res["gemm_status"] = gemm_status()
    if rank == 0:
        print(json.dumps(res), flush=True)
    if world > 1:
        dist.barrier()
    comm.destroy()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
