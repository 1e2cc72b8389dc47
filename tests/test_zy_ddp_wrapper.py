"""The data-parallel wrapper on one GPU: gradients live in flat buckets, every bucket is reduced by
ONE launch of the library's fused scale / cast kernel as soon as its last gradient is ready, and the
fp32 main gradients equal the bf16 gradients (world size 1: the sum of one operand)."""
import pytest

torch = pytest.importorskip("torch")

pytestmark = pytest.mark.gpu


def _tiny_model():
    from mini_nccl_b200.models import GPT2Config, GPT2Model

    cfg = GPT2Config.tiny()
    torch.manual_seed(0)
    return cfg, GPT2Model(cfg).cuda().to(torch.bfloat16)


def test_buckets_hooks_and_fused_cast_single_rank():
    import mini_nccl_b200 as mn
    from mini_nccl_b200.parallel import DistributedDataParallel

    cfg, model = _tiny_model()
    comm = mn.Communicator(1, 0)
    try:
        ddp = DistributedDataParallel(model, comm, bucket_mb=0.25, main_grad_dtype=torch.float32)
        assert len(ddp.buckets) > 1, "0.25 MB buckets must split the tiny model"
        # gradients are views into the buckets
        for b in ddp.buckets:
            lo, hi = b.flat.data_ptr(), b.flat.data_ptr() + b.flat.numel() * b.flat.element_size()
            assert all(lo <= p.grad.data_ptr() < hi for p in b.params)
        ids = torch.randint(0, cfg.vocab_size, (2, cfg.seq_len), device="cuda")
        for step in range(2):
            ddp.zero_grad()
            before = ddp.launches
            loss = ddp(ids, ids)
            loss.backward()
            torch.cuda.synchronize()
            assert torch.isfinite(loss).item()
            assert ddp.launches - before == len(ddp.buckets), "one launch per bucket and step"
            for b in ddp.buckets:
                assert torch.equal(b.main, b.flat.float()), "fused cast kernel produced wrong main gradients"
            assert any(p.grad.abs().sum().item() > 0 for p in model.parameters())
        assert comm.stats()["algo"]["local"] == ddp.launches
    finally:
        comm.destroy()


def test_reduction_after_backward_when_overlap_is_off():
    import mini_nccl_b200 as mn
    from mini_nccl_b200.parallel import DistributedDataParallel

    cfg, model = _tiny_model()
    comm = mn.Communicator(1, 0)
    try:
        ddp = DistributedDataParallel(model, comm, bucket_mb=0.25, main_grad_dtype=torch.float32, overlap=False)
        ids = torch.randint(0, cfg.vocab_size, (2, cfg.seq_len), device="cuda")
        loss = ddp(ids, ids)
        loss.backward()
        torch.cuda.synchronize()
        assert ddp.launches == len(ddp.buckets)
        for b in ddp.buckets:
            assert torch.equal(b.main, b.flat.float())
    finally:
        comm.destroy()
