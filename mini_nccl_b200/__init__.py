"""mini_nccl_b200: a Blackwell-native collective-communication library with the
capabilities and C ABI of Mini-NCCL, plus a thin PyTorch binding.

Layout:
  _lib        ctypes binding to libmini_nccl.so (built in-tree by ``build``)
  comm        Communicator (tensor AllReduce / ReduceScatter / AllGather, symmetric tensors)
  parallel    DDP wrapper + gradient hook, tensor-parallel MLP block
  ops         sm_100a tcgen05 GEMM and the fused GEMM+collective kernels
  models      GPT-2 shaped decoder, Llama-3 shaped MLP block (benchmark workloads)
  utils       timing, clock sampling, host oracles
"""
from ._lib import (ALGO_NAMES, AVG, BFLOAT16, FLOAT16, FLOAT32, FLOAT64, INT8, INT32, INT64, MAX, MIN, PROD, SUM, UINT8,
                   UINT32, UINT64, MiniNcclError, lib, lib_file)
from .comm import Communicator

__all__ = ["Communicator", "MiniNcclError", "lib", "lib_file"]
__version__ = "0.1.0"


def __getattr__(name):
    # Submodules on first use (`mn.ops.gemm_bf16`, `mn.parallel.DistributedDataParallel`, ...): they pull in
    # torch, which the ctypes binding itself does not need.
    if name in ("ops", "parallel", "models", "utils", "build"):
        import importlib

        return importlib.import_module("." + name, __name__)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
