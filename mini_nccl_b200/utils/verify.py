"""Correctness battery against the host oracle, for real multi-process runs.

The reference's benchmark verifies every size it times (reference: tests/perf_test.cpp:102-134),
but against a constant.  This battery runs every AllReduce algorithm of the library through the
real multi-process path on seeded random inputs (seed + rank), on symmetric and on ordinary
buffers, fp32 and bf16, with one small and one large element count that the rank count does not
divide, and compares with the rank-ordered host oracle:

* peer-to-peer algorithms (LL, one-shot, two-shot, staged, the stream pipeline): bit for bit;
* NVLS and the pipelined kernel where it reduces through the switch (the switch defines the order
  of the sum): within a tolerance on random data, and bit for bit on exactly representable data
  (small integers), where the order cannot matter;
* the two fused GEMM kernels on a small shape: bit for bit on integer-valued operands (every
  product and sum is exact in fp32 whatever the tensor cores' order), within a tolerance on random
  operands.  Where GEMM -> reduce-scatter lets the switch add the partial tiles, a sum that lies
  exactly halfway between two bf16 values may be rounded to either neighbour (the switch does not
  round ties to even): the other neighbour is accepted there and nowhere else.

Every rank regenerates every rank's input from the seeds, so no data is exchanged for checking.
"""
from __future__ import annotations

import numpy as np

from .. import _lib
from . import oracle as O


def _torch_dt(code):
    import torch

    return {_lib.FLOAT32: torch.float32, _lib.BFLOAT16: torch.bfloat16}[code]


def _to_device(bits: np.ndarray, code: int, out):
    """Host array in the oracle's storage type -> the given device tensor."""
    import torch

    if code == _lib.BFLOAT16:
        out.view(torch.int16).copy_(torch.from_numpy(bits.view(np.int16)))
    else:
        out.copy_(torch.from_numpy(bits))
    return out


def _to_host(t, code: int) -> np.ndarray:
    import torch

    if code == _lib.BFLOAT16:
        return t.view(torch.int16).cpu().numpy().view(np.uint16)
    return t.cpu().numpy()


def _exact_input(code: int, count: int, rank: int) -> np.ndarray:
    """Small integers: sums of up to 16 of them are exact in bf16 and fp32 in any order."""
    rng = np.random.default_rng(777 + rank)
    x = rng.integers(-7, 8, count).astype(np.float32)
    return O.f32_to_bf16_bits(x) if code == _lib.BFLOAT16 else x


def check_allreduce(comm, world: int, rank: int, small: int = 2051, large: int = (16 << 20) + 5,
                    dtypes=(_lib.FLOAT32, _lib.BFLOAT16)) -> dict:
    """Runs the battery; returns {"cases", "failed", "nvls", "failures": [...], "algos": {...}}."""
    import torch

    res = {"cases": 0, "failed": 0, "nvls": False, "failures": [], "algos": {}}
    if world == 1:
        # one rank: out = scale * in, out of place
        for code in dtypes:
            x = O.make_input(code, small, 0, dist="normal")
            t = _to_device(x, code, torch.empty(small, dtype=_torch_dt(code), device="cuda"))
            out = torch.empty_like(t)
            comm.all_reduce(t, "sum", out=out, scale=0.5)
            torch.cuda.synchronize()
            want = O.oracle_allreduce([x], code, _lib.SUM, scale=0.5)
            res["cases"] += 1
            if not np.array_equal(_to_host(out, code), want):
                res["failed"] += 1
                res["failures"].append("local %s" % O.DTYPE_NAMES[code])
        return res

    scale = 1.0 / world
    for code in dtypes:
        dt = _torch_dt(code)
        esz = _lib.DTYPE_SIZES[code]
        for count, algos in ((small, ("ll", "oneshot", "twoshot", "nvls")), (large * (4 // esz), ("twoshot", "nvls", "pipe", "auto"))):
            inputs = [O.make_input(code, count, r, dist="normal") for r in range(world)]
            want = O.oracle_allreduce(inputs, code, _lib.SUM, scale=scale)
            exact_in = [_exact_input(code, count, r) for r in range(world)]
            exact_want = O.oracle_allreduce(exact_in, code, _lib.SUM, scale=1.0)
            tol = O.tolerance(code, world) * scale
            sym = comm.empty(count, dt)
            plain = torch.empty(count, dtype=dt, device="cuda")
            plain_out = torch.empty(count, dtype=dt, device="cuda")
            for where, src, dst in (("symmetric", sym, sym), ("ordinary", plain, plain_out)):
                for algo in algos:
                    if algo in ("auto", "pipe") and where == "symmetric":
                        continue  # auto: same kernel as the forced ones; pipe: a kernel for ordinary buffers
                    before = comm.stats().get("algo", {})
                    _to_device(inputs[rank], code, src)
                    comm.all_reduce(src, "sum", out=dst, scale=scale, algo=algo)
                    torch.cuda.synchronize()
                    got = _to_host(dst, code)
                    after = comm.stats().get("algo", {})
                    used = [k for k in after if after[k] != before.get(k, 0)]
                    # the pipelined kernel reduces through the switch too where the communicator has one
                    # (more than two ranks): its sum is ordered by the switch, like the NVLS kernel's
                    switch = "nvls" in used or ("pipe" in used and world > 2 and bool(comm.stats().get("nvls")))
                    name = "%s/%s/%s/%d" % (algo, where, O.DTYPE_NAMES[code], count)
                    res["algos"][name] = "+".join(used)
                    res["cases"] += 1
                    if switch:
                        res["nvls"] = True
                        ok = bool(np.all(np.abs(O.to_float64(got, code) - O.to_float64(want, code)) <= tol))
                        # and bit for bit where the order of the sum cannot matter
                        _to_device(exact_in[rank], code, src)
                        comm.all_reduce(src, "sum", out=dst, algo=algo)
                        torch.cuda.synchronize()
                        res["cases"] += 1
                        if not np.array_equal(_to_host(dst, code), exact_want):
                            res["failed"] += 1
                            res["failures"].append(name + " (exact data)")
                    else:
                        ok = bool(np.array_equal(got, want))
                    if not ok:
                        res["failed"] += 1
                        bad = int(np.count_nonzero(got != want))
                        res["failures"].append("%s: %d elements differ" % (name, bad))
            comm.free(sym)
            del plain, plain_out
    return res


def switch_ties(got_bits: np.ndarray, want_bits: np.ndarray, exact_sum: np.ndarray) -> np.ndarray:
    """Where a result differs from the oracle's only because the NVSwitch rounded a tie the other way.

    The switch adds the bf16 partial sums in fp32 (exact for the integer operands of the check) and
    rounds once, but not to nearest-even: a sum that lies exactly halfway between two bf16 values may
    land on either neighbour.  True exactly where ``got`` and ``want`` differ and both are equally far
    from the exact sum; any other difference stays a failure."""
    exact = np.asarray(exact_sum, dtype=np.float64)
    d_got = np.abs(O.bf16_bits_to_f32(got_bits).astype(np.float64) - exact)
    d_want = np.abs(O.bf16_bits_to_f32(want_bits).astype(np.float64) - exact)
    return (got_bits != want_bits) & (d_got == d_want) & (d_got > 0)


def check_fused_gemm(comm, world: int, rank: int, M: int = 1024, N: int = 1024, K: int = 512) -> dict:
    """GEMM -> reduce-scatter and all-gather -> GEMM on a small shape against the host restatements."""
    import torch

    from ..ops import AllGatherGemm, GemmReduceScatter, gemm_status

    res = {"cases": 0, "failed": 0, "failures": []}
    per = M // world
    if M % world or per % 128:
        return res
    rs = GemmReduceScatter(comm, M, N)
    ag = AllGatherGemm(comm, M, K)

    def bits_to_dev(b):
        return torch.from_numpy(b.view(np.int16)).cuda().view(torch.bfloat16)

    for kind in ("exact", "random"):
        def operands(r):
            rng = np.random.default_rng(4242 + r + (0 if kind == "exact" else 100))
            if kind == "exact":
                gen = lambda *s: rng.integers(-2, 3, s).astype(np.float32)
            else:
                gen = lambda *s: rng.standard_normal(s).astype(np.float32)
            return O.f32_to_bf16_bits(gen(M, K)), O.f32_to_bf16_bits(gen(N, K)), O.f32_to_bf16_bits(gen(per, K))

        ops = [operands(r) for r in range(world)]
        want, want_sum = O.oracle_gemm_reduce_scatter([o[0] for o in ops], [o[1] for o in ops], rank, return_sum=True)
        out = rs(bits_to_dev(ops[rank][0]), bits_to_dev(ops[rank][1]))
        torch.cuda.synchronize()
        got = out.view(torch.int16).cpu().numpy().view(np.uint16)
        res["cases"] += 1
        if gemm_status() != 0:
            res["failed"] += 1
            res["failures"].append("gemm_rs/%s: a bounded wait ran out" % kind)
        elif kind == "exact":
            bad = got != want
            if rs.in_switch and bad.any():
                tie = switch_ties(got, want, want_sum)
                if tie.any():
                    res.setdefault("notes", []).append("gemm_rs/exact: %d of %d sums are ties that the switch rounded to the "
                                                       "other neighbour" % (int(tie.sum()), tie.size))
                bad = bad & ~tie
            if bad.any():
                res["failed"] += 1
                res["failures"].append("gemm_rs/exact: %d elements differ" % int(np.count_nonzero(bad)))
        else:
            w = O.bf16_bits_to_f32(want)
            err = float(np.abs(O.bf16_bits_to_f32(got) - w).max() / max(np.abs(w).max(), 1e-30))
            if err > 1e-2:
                res["failed"] += 1
                res["failures"].append("gemm_rs/random: rel err %.3g" % err)
        gathered, want2 = O.oracle_all_gather_gemm([o[2] for o in ops], ops[rank][1])
        ag.local_shard.copy_(bits_to_dev(ops[rank][2]))
        c = ag(bits_to_dev(ops[rank][1]))
        torch.cuda.synchronize()
        got2 = c.view(torch.int16).cpu().numpy().view(np.uint16)
        got_g = ag.gather.view(torch.int16).cpu().numpy().view(np.uint16)
        res["cases"] += 1
        if gemm_status() != 0:
            res["failed"] += 1
            res["failures"].append("ag_gemm/%s: a bounded wait ran out" % kind)
        elif not np.array_equal(got_g, gathered):
            res["failed"] += 1
            res["failures"].append("ag_gemm/%s: gathered rows differ" % kind)
        elif kind == "exact":
            if not np.array_equal(got2, want2):
                res["failed"] += 1
                res["failures"].append("ag_gemm/exact: %d elements differ" % int(np.count_nonzero(got2 != want2)))
        else:
            w = O.bf16_bits_to_f32(want2)
            err = float(np.abs(O.bf16_bits_to_f32(got2) - w).max() / max(np.abs(w).max(), 1e-30))
            if err > 1e-2:
                res["failed"] += 1
                res["failures"].append("ag_gemm/random: rel err %.3g" % err)
    return res
