"""The sm_100a tcgen05 GEMM against a plain PyTorch fp32 reference of the same product."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _check(M, N, K, out_dtype=torch.bfloat16, lda_pad=0):
    from mini_nccl_b200.ops import gemm_bf16, gemm_status

    g = torch.Generator(device="cuda").manual_seed(M * 7 + N * 3 + K)
    a_full = torch.randn(M, K + lda_pad, generator=g, device="cuda").to(torch.bfloat16)
    a = a_full[:, :K]
    b = torch.randn(N, K, generator=g, device="cuda").to(torch.bfloat16)
    c = gemm_bf16(a, b, out_dtype=out_dtype)
    assert gemm_status() == 0, "a bounded wait ran out inside the GEMM"
    ref = a.float() @ b.float().t()
    err = (c.float() - ref).abs().max().item()
    scale = ref.abs().max().item() + 1e-6
    tol = 2e-2 if out_dtype == torch.bfloat16 else 2e-4
    assert err / scale < tol, f"M={M} N={N} K={K}: max err {err} (scale {scale})"


@pytest.fixture(params=[0, 1], ids=["single_cta", "cta_pair"], autouse=True)
def kernel_choice(request):
    """Every GEMM test runs on the single-CTA kernel and on the CTA-pair (cta_group::2) kernel."""
    from mini_nccl_b200.ops.gemm import set_pair_mode

    set_pair_mode(request.param)
    yield request.param
    set_pair_mode(-1)


def test_gemm_single_tile():
    _check(128, 256, 64)
    _check(128, 256, 256)


def test_gemm_fp32_output_is_exact_to_accumulation():
    _check(256, 512, 512, out_dtype=torch.float32)


def test_gemm_multi_tile_persistent():
    _check(1024, 1024, 1024)
    _check(4096, 3584, 4096)     # all-gather -> GEMM shape of the tensor-parallel block (per rank)
    _check(4096, 4096, 1792)     # GEMM -> reduce-scatter shape


def test_gemm_ragged_edges_and_strides():
    _check(100, 200, 72)         # partial tiles in M and N, K not a multiple of 64
    _check(300, 264, 136, out_dtype=torch.float32)
    _check(257, 520, 64, lda_pad=8)


def test_gemm_many_more_tiles_than_sms():
    _check(8192, 4096, 512)


def test_fused_kernels_single_rank():
    # One rank: the same kernels run locally (push to the own staging slot, reduce one slot; no
    # communication CTAs).  Checks the epilogue hooks, the epochs over repeated calls and the
    # staging halves.
    import mini_nccl_b200 as mn
    from mini_nccl_b200.ops import AllGatherGemm, GemmReduceScatter, gemm_status

    comm = mn.Communicator(1, 0)
    try:
        M, N, K = 512, 1024, 384
        rs = GemmReduceScatter(comm, M, N)
        ag = AllGatherGemm(comm, M, K)
        for it in range(3):
            g = torch.Generator(device="cuda").manual_seed(it)
            a = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
            b = torch.randn(N, K, generator=g, device="cuda").to(torch.bfloat16)
            ref = a.float() @ b.float().t()
            out = rs(a, b)
            assert gemm_status() == 0
            assert (out.float() - ref).abs().max().item() / ref.abs().max().item() < 2e-2
            ag.local_shard.copy_(a)
            c = ag(b)
            assert gemm_status() == 0
            assert (c.float() - ref).abs().max().item() / ref.abs().max().item() < 2e-2
    finally:
        comm.destroy()
