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


def test_gemm_large_k_fp32_output_tight():
    # fp32 output shows the accumulator itself: a dropped or doubled 64-wide k-block moves an element by
    # ~K^-1/2 of the scale (1.5 % at K = 4096), a hundred times this bound.
    _check(4096, 3584, 4096, out_dtype=torch.float32)
    _check(4096, 4096, 1792, out_dtype=torch.float32)


def test_gemm_integer_operands_bit_exact():
    """Small integers: every product and every partial sum is exact in fp32 whatever the order, so the
    result must equal the host product bit for bit (bf16 output: one rounding of an exact sum)."""
    import numpy as np

    from mini_nccl_b200.ops import gemm_bf16, gemm_status
    from mini_nccl_b200.utils import oracle as O

    rng = np.random.default_rng(11)
    M, N, K = 384, 512, 4096
    a = O.f32_to_bf16_bits(rng.integers(-3, 4, (M, K)).astype(np.float32))
    b = O.f32_to_bf16_bits(rng.integers(-3, 4, (N, K)).astype(np.float32))
    want = O.oracle_gemm_bf16(a, b)
    want32 = O.oracle_gemm_bf16(a, b, out_fp32=True)
    da = torch.from_numpy(a.view(np.int16)).cuda().view(torch.bfloat16)
    db = torch.from_numpy(b.view(np.int16)).cuda().view(torch.bfloat16)
    got = gemm_bf16(da, db).view(torch.int16).cpu().numpy().view(np.uint16)
    got32 = gemm_bf16(da, db, out_dtype=torch.float32).cpu().numpy()
    assert gemm_status() == 0
    assert np.array_equal(got, want)
    assert np.array_equal(got32, want32)


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


def test_fused_kernels_single_rank_bit_exact_against_the_host_oracle():
    """Integer-valued operands: both fused kernels must reproduce the host restatement bit for bit
    (the rounding of every partial tile to bf16 before it travels included)."""
    import mini_nccl_b200 as mn
    from mini_nccl_b200.utils import verify

    comm = mn.Communicator(1, 0)
    try:
        res = verify.check_fused_gemm(comm, 1, 0, M=512, N=1024, K=512)
        assert res["cases"] == 4 and res["failed"] == 0, res["failures"]
    finally:
        comm.destroy()


@pytest.mark.parametrize("M,F,K", [(256, 128, 192), (512, 1792, 512), (384, 272, 128)])
def test_all_gather_gemm_with_swiglu_in_the_epilogue(M, F, K):
    """act = silu(X Wg^T) * (X Wu^T) out of ONE kernel (weights interleaved in groups of 16 rows) against a
    plain PyTorch fp32 computation; the (gate | up) matrix is never written."""
    import mini_nccl_b200 as mn
    from mini_nccl_b200.ops import AllGatherGemm, gemm_status, interleave_gate_up, split_gate_up

    comm = mn.Communicator(1, 0)
    try:
        g = torch.Generator(device="cuda").manual_seed(M + F + K)
        x = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
        wg = (torch.randn(F, K, generator=g, device="cuda") * 0.2).to(torch.bfloat16)
        wu = (torch.randn(F, K, generator=g, device="cuda") * 0.2).to(torch.bfloat16)
        w = interleave_gate_up(wg, wu)
        gate_cols, up_cols = split_gate_up(w.t().contiguous())          # the helper pair round-trips
        assert torch.equal(gate_cols.t(), wg) and torch.equal(up_cols.t(), wu)
        ag = AllGatherGemm(comm, M, K)
        ag.local_shard.copy_(x)
        out_big = torch.zeros(M, F + 8, device="cuda", dtype=torch.bfloat16)
        act = ag(w, out=out_big[:, :F], swiglu=True)
        torch.cuda.synchronize()
        assert gemm_status() == 0
        gt, ut = x.float() @ wg.float().t(), x.float() @ wu.float().t()
        ref = gt * torch.sigmoid(gt) * ut
        err = (act.float() - ref).abs()
        # one rounding to bf16 of an fp32 result whose inputs carry the tensor cores' summation order
        assert torch.all(err <= ref.abs() * 2.0 ** -6 + 2e-2 * ref.abs().max() * 2.0 ** -6), float(err.max())
        assert torch.count_nonzero(out_big[:, F:]) == 0, "columns outside the output view were written"
        # the plain product with the same weights still works after a SwiGLU call (shared buffers, epochs)
        h = ag(w)
        torch.cuda.synchronize()
        g2, u2 = split_gate_up(h)
        assert (g2.float() - gt).abs().max().item() / gt.abs().max().item() < 2e-2
        assert (u2.float() - ut).abs().max().item() / ut.abs().max().item() < 2e-2
    finally:
        comm.destroy()



def test_fused_kernel_wait_is_bounded_and_reports_to_the_communicator():
    """The wait the fused kernels use for a peer, on a flag that nothing sets: it gives up after its
    budget (or at once when the abort word is set), and the failure reaches the communicator's status
    words, from where the watchdog fails the communicator.  A failure made on the host; nothing faults."""
    import ctypes as C

    import mini_nccl_b200 as mn

    L = mn.lib()
    st, us, words = C.c_uint32(), C.c_uint32(), (C.c_uint32 * 4)()
    assert L.mncclGemmProbeFlagWait(50_000_000, 0, C.byref(st), C.byref(us), words) == 0   # 50 ms budget
    assert st.value == 3, "flag wait timed out"
    assert 40_000 <= us.value < 2_000_000, us.value
    assert words[0] == 1 and (words[1] & 0xffff) == (0x8000 | 3), "status = timeout, detail names the code"
    assert words[2] == 1, "the kernel counted itself as started"
    assert L.mncclGemmProbeFlagWait(2_000_000_000, 1, C.byref(st), C.byref(us), words) == 0
    assert st.value == 4 and us.value < 100_000, "abort word set: the wait returns at once"
    assert words[0] == 2, "status = aborted"
