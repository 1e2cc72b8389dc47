"""Hand-written sm_100a compute kernels: the tcgen05 / TMEM / TMA bf16 GEMM and its fusions
with the collectives (GEMM -> reduce-scatter, all-gather -> GEMM)."""
from .gemm import gemm_bf16, gemm_status  # noqa: F401
from .fused import AllGatherGemm, GemmReduceScatter, interleave_gate_up, split_gate_up  # noqa: F401,E402
from .elementwise import swiglu_bf16  # noqa: F401,E402
