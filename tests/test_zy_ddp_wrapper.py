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


def test_stock_optimizer_zero_grad_and_no_sync():
    """optimizer.zero_grad() with its default set_to_none=True makes autograd allocate fresh .grad tensors:
    the wrapper must move them back into the buckets (what gets reduced is the bucket).  Under no_sync() the
    backward only accumulates; the next synchronised backward reduces the sum."""
    import mini_nccl_b200 as mn
    from mini_nccl_b200.parallel import DistributedDataParallel

    cfg, model = _tiny_model()
    comm = mn.Communicator(1, 0)
    try:
        ddp = DistributedDataParallel(model, comm, bucket_mb=0.25, main_grad_dtype=torch.float32)
        opt = torch.optim.SGD(model.parameters(), lr=1e-3)
        ids = torch.randint(0, cfg.vocab_size, (2, cfg.seq_len), device="cuda")
        used = lambda: [p for p in model.parameters() if p.grad is not None]
        for step in range(2):
            opt.zero_grad()                      # default arguments: .grad becomes None
            assert all(p.grad is None for p in model.parameters())
            ddp(ids, ids).backward()
            torch.cuda.synchronize()
            assert ddp.repaired > 0
            for b in ddp.buckets:
                lo, hi = b.flat.data_ptr(), b.flat.data_ptr() + b.flat.numel() * b.flat.element_size()
                assert all(p.grad is not None and lo <= p.grad.data_ptr() < hi for p in b.params), "a .grad left its bucket"
                assert torch.equal(b.main, b.flat.float()), "the reduced bucket does not hold this step's gradients"
            assert any(p.grad.abs().sum().item() > 0 for p in used())
            opt.step()
        # gradient accumulation: two micro-steps, one reduction
        ddp.zero_grad()
        before = ddp.launches
        with ddp.no_sync():
            ddp(ids, ids).backward()
        torch.cuda.synchronize()
        assert ddp.launches == before, "no collective under no_sync()"
        once = [b.flat.clone() for b in ddp.buckets]
        ddp(ids, ids).backward()
        torch.cuda.synchronize()
        assert ddp.launches - before == len(ddp.buckets)
        for b, o in zip(ddp.buckets, once):
            assert torch.allclose(b.flat.float(), 2 * o.float(), rtol=2e-2, atol=1e-3), "second micro-step did not accumulate"
            assert torch.equal(b.main, b.flat.float())
    finally:
        comm.destroy()
