"""Pinned host buffers on one GPU: the reference's programs hand pinned host memory to
ncclAllReduce (src/main.cpp:35, tests/perf_test.cpp:78-79).  From a few megabytes up the copy
engines move such buffers in chunks (host -> device, kernel, device -> host as a pipeline);
the result must equal a plain PyTorch fp32 computation."""
import pytest

torch = pytest.importorskip("torch")

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def comm():
    import mini_nccl_b200 as mn

    c = mn.Communicator(1, 0)
    yield c
    c.destroy()


def test_host_in_host_out_scaled(comm):
    n = (5 << 20) + 777                       # 20 MB: three chunks of 8 MB, ragged tail
    x = torch.randn(n).pin_memory()
    y = torch.zeros(n).pin_memory()
    before = comm.stats()["pipelined_calls"]
    comm.all_reduce(x, "sum", out=y, scale=0.5)
    torch.cuda.synchronize()
    assert torch.equal(y, x * 0.5)
    assert comm.stats()["pipelined_calls"] == before + 1


def test_host_in_place(comm):
    n = 3 << 20
    x = torch.randn(n).pin_memory()
    ref = x.clone()
    comm.all_reduce(x, "sum", scale=2.0)
    torch.cuda.synchronize()
    assert torch.equal(x, ref * 2.0)


def test_host_to_device_and_back_with_cast(comm):
    n = (4 << 20) + 64
    x = torch.randn(n).pin_memory()
    d = torch.zeros(n, dtype=torch.bfloat16, device="cuda")
    comm.all_reduce(x, "sum", out=d)          # pinned fp32 -> device bf16
    torch.cuda.synchronize()
    assert torch.equal(d.cpu(), x.to(torch.bfloat16))
    h = torch.zeros(n).pin_memory()
    comm.all_reduce(d, "sum", out=h)          # device bf16 -> pinned fp32
    torch.cuda.synchronize()
    assert torch.equal(h, x.to(torch.bfloat16).float())


def test_small_host_buffer_takes_the_direct_kernel(comm):
    x = torch.randn(1000).pin_memory()
    y = torch.zeros(1000).pin_memory()
    before = comm.stats()["pipelined_calls"]
    comm.all_reduce(x, "sum", out=y)
    torch.cuda.synchronize()
    assert torch.equal(y, x)
    assert comm.stats()["pipelined_calls"] == before


def test_host_pipeline_in_cuda_graph(comm):
    n = 3 << 20
    x = torch.randn(n).pin_memory()
    y = torch.zeros(n).pin_memory()
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        comm.all_reduce(x, "sum", out=y, scale=3.0)   # warm-up outside capture (allocates the staging)
        s.synchronize()
        with torch.cuda.graph(g, stream=s):
            comm.all_reduce(x, "sum", out=y, scale=3.0)
    y.zero_()
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(y, x * 3.0)
