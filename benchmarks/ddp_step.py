"""Data-parallel training step of a GPT-2-medium shaped decoder (24 layers, d_model 1024, 16 heads,
vocabulary 50257, sequence 1024, micro-batch 8 per GPU, bf16 weights, random init, synthetic token
ids): this library's DDP wrapper (25 MB buckets in symmetric memory, AllReduce fused with the
1/world scale, overlapped with backward) against torch DistributedDataParallel over NCCL.
A step is forward + backward + gradient AllReduce + fused AdamW.  Device-timed, max over ranks.

  python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/ddp_step.py
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def main():
    import torch
    import torch.distributed as dist

    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=24)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--impl", default="both", choices=["both", "ours", "torch"])
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MINI_NCCL_BOOTSTRAP_PORT", str(int(os.environ.get("MASTER_PORT", "29500")) + 17))
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    import mini_nccl_b200 as mn
    from mini_nccl_b200.models import GPT2Config, GPT2Model
    from mini_nccl_b200.parallel import DistributedDataParallel
    from mini_nccl_b200.utils.timing import max_over_ranks

    cfg = GPT2Config(n_layer=args.layers)
    tokens_per_step = args.batch * cfg.seq_len * world
    res = {"world": world, "model": f"gpt2-medium-shaped ({args.layers} layers)", "micro_batch": args.batch,
           "seq_len": cfg.seq_len, "tokens_per_step": tokens_per_step}

    def run(kind):
        torch.manual_seed(0)
        model = GPT2Model(cfg).cuda().to(torch.bfloat16)
        comm = None
        if kind == "ours":
            comm = mn.Communicator(world, rank, os.environ["MASTER_ADDR"])
            wrapped = DistributedDataParallel(model, comm, bucket_mb=25.0)
        elif world > 1:
            wrapped = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local_rank], bucket_cap_mb=25,
                                                                gradient_as_bucket_view=True)
        else:
            wrapped = model
        opt = torch.optim.AdamW(model.parameters(), lr=1e-4, fused=True)
        gen = torch.Generator(device="cuda").manual_seed(1234 + rank)
        ids = torch.randint(0, cfg.vocab_size, (args.batch, cfg.seq_len), generator=gen, device="cuda")

        def step():
            if kind == "ours":
                wrapped.zero_grad()
            else:
                opt.zero_grad(set_to_none=False)
            loss = wrapped(ids, ids)
            loss.backward()
            opt.step()
            return loss

        for _ in range(args.warmup):
            loss = step()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            loss = step()
        e1.record()
        torch.cuda.synchronize()
        ms = max_over_ranks(e0.elapsed_time(e1) / args.steps)
        out = {"ms_per_step": round(ms, 2), "tokens_per_s": round(tokens_per_step / ms * 1e3, 1), "loss": round(float(loss), 4)}
        if kind == "ours":
            out["buckets"] = len(wrapped.buckets)
            out["bucket_mb"] = [round(b / 2 ** 20, 1) for b in wrapped.bucket_bytes()][:4]
            out["algo"] = comm.stats()["algo"]
            del wrapped, opt
            comm.destroy()
        return out

    if args.impl in ("both", "torch"):
        res["torch_ddp_nccl"] = run("torch")
    if args.impl in ("both", "ours"):
        res["ours"] = run("ours")
    if "ours" in res and "torch_ddp_nccl" in res:
        res["speedup"] = round(res["torch_ddp_nccl"]["ms_per_step"] / res["ours"]["ms_per_step"], 4)
    if rank == 0:
        print(json.dumps(res), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
