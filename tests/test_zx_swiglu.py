"""The one-pass SwiGLU kernel of the tensor-parallel block against a plain PyTorch fp32 computation of
the same operation (runs late in the suite: it is the newest kernel)."""
import pytest

torch = pytest.importorskip("torch")

pytestmark = pytest.mark.gpu


def _reference(h):
    f = h.shape[1] // 2
    g, u = h[:, :f].float(), h[:, f:].float()
    return (g * torch.sigmoid(g) * u)


@pytest.mark.parametrize("m,f", [(1, 8), (37, 72), (512, 1792), (4096, 1792)])
def test_swiglu_matches_fp32_reference(m, f):
    from mini_nccl_b200.ops import swiglu_bf16

    torch.manual_seed(m * 131 + f)
    h = (torch.randn(m, 2 * f, device="cuda") * 2.0).to(torch.bfloat16)
    out = swiglu_bf16(h)
    torch.cuda.synchronize()
    ref = _reference(h)
    # one rounding to bf16 (2^-8 relative); __expf adds a few ulp of fp32, far below that
    err = (out.float() - ref).abs()
    assert torch.all(err <= ref.abs() * 2.0 ** -7 + 1e-6), float(err.max())


def test_swiglu_strided_rows_and_argument_checks():
    from mini_nccl_b200.ops import swiglu_bf16

    big = (torch.randn(64, 512, device="cuda")).to(torch.bfloat16)
    h = big[:, :256]                      # row stride 512, F = 128
    out_big = torch.zeros(64, 256, device="cuda", dtype=torch.bfloat16)
    out = out_big[:, :128]                # row stride 256
    swiglu_bf16(h, out=out)
    torch.cuda.synchronize()
    ref = _reference(h)
    assert torch.all((out.float() - ref).abs() <= ref.abs() * 2.0 ** -7 + 1e-6)
    assert torch.count_nonzero(out_big[:, 128:]) == 0, "columns outside the output view were written"
    with pytest.raises(TypeError):
        swiglu_bf16(big.float())
    with pytest.raises(RuntimeError):
        swiglu_bf16(torch.zeros(4, 12, device="cuda", dtype=torch.bfloat16))   # F = 6 is no multiple of 8
