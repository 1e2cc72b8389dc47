"""bf16 GEMM throughput: the hand-written tcgen05 kernel against cuBLAS (torch.matmul) on the
shapes of the tensor-parallel block.  CUDA events, warm-up, L2 flushed between timed calls by
writing a 256 MB buffer; the kernels take turns inside each iteration and medians are reported; fractions are of the measured cuBLAS peak in MEASURED_PEAKS.json."""
from __future__ import annotations

import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def time_ops(fns, iters=20, flush=None):
    """Median device time (ms) of each callable; the callables take turns inside every iteration, so
    that clock and temperature drift hits all of them alike."""
    import torch

    for fn in fns:
        for _ in range(3):
            fn()
    torch.cuda.synchronize()
    samples = [[] for _ in fns]
    for _ in range(iters):
        for i, fn in enumerate(fns):
            if flush is not None:
                flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            samples[i].append(e0.elapsed_time(e1))
    return [sorted(x)[len(x) // 2] for x in samples]


def main():
    import torch

    from mini_nccl_b200.ops import gemm_bf16, gemm_status
    from mini_nccl_b200.ops.gemm import set_pair_mode

    peak = 1590.0
    try:
        peak = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"]
    except Exception:
        pass
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    shapes = [(4096, 3584, 4096), (4096, 4096, 1792), (4096, 4096, 512), (8192, 8192, 8192), (1024, 1024, 1024),
              (8192, 4096, 4096), (16384, 8192, 4096), (2048, 2048, 8192), (4096, 14336, 4096)]
    import ctypes
    import mini_nccl_b200 as mn
    L = mn.lib()
    L.mncclGemmMaxPairs.restype = ctypes.c_int
    print(json.dumps({"max_resident_cta_pairs": L.mncclGemmMaxPairs()}), flush=True)
    rows = []
    for M, N, K in shapes:
        a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
        b = torch.randn(N, K, device="cuda").to(torch.bfloat16)
        c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        def run(mode):
            set_pair_mode(mode)
            gemm_bf16(a, b, out=c)

        ms_single, ms_pair, ms_ours, ms_lib = time_ops(
            [lambda: run(0), lambda: run(1), lambda: run(-1), lambda: torch.matmul(a, b.t(), out=c)], flush=flush)
        set_pair_mode(-1)
        fl = 2.0 * M * N * K
        row = {"M": M, "N": N, "K": K, "ours_us": round(ms_ours * 1e3, 1), "single_cta_us": round(ms_single * 1e3, 1), "cta_pair_us": round(ms_pair * 1e3, 1), "cublas_us": round(ms_lib * 1e3, 1),
               "ours_tflops": round(fl / ms_ours / 1e9, 1), "cublas_tflops": round(fl / ms_lib / 1e9, 1),
               "ours_frac_of_measured_peak": round(fl / ms_ours / 1e9 / peak, 3), "status": gemm_status()}
        rows.append(row)
        print(json.dumps(row), flush=True)
    return rows


if __name__ == "__main__":
    main()
