"""Parallelism built on the communicator: data parallel (bucketed, overlapped, fused
scale / cast AllReduce) and tensor parallel (GEMM -> reduce-scatter, all-gather -> GEMM)."""
from .ddp import DistributedDataParallel, allreduce_comm_hook  # noqa: F401
from .tp import TensorParallelAttnOut, TensorParallelMLP  # noqa: F401,E402
