"""The two tensor-parallel fusions as Python objects that own their workspaces.

``GemmReduceScatter``: ``out[M/R, N] = reduce_scatter(A_r[M, K_r] @ B_r[N, K_r].T)`` -- one kernel.
Where the NVSwitch can reduce (NVLS), the partial tiles stay on their rank and the owner of a row block
sums all ranks' copies in the switch (``multimem.ld_reduce``) while the remaining tiles are computed;
otherwise (no multicast mapping, ``MINI_NCCL_NVLS_ENABLE=0``, ``MINI_NCCL_RS_SWITCH=0``, or more than four
ranks unless ``MINI_NCCL_RS_SWITCH=1``: that size has not been measured) tiles are pushed to their owner
over NVLink and summed there in rank order.
``AllGatherGemm``: ``C[M, N_r] = all_gather(X_r)[M, K] @ B_r[N_r, K].T`` -- one kernel; a few CTAs push
the local shard to the peers while the others already compute on the local rows.

Workspaces come from ``Communicator.empty`` (symmetric memory), so creating these objects is
collective: every rank, same order, same shapes.  With one rank they run the same kernels locally.

Both kernels run under the communicator's failure model: every wait on a peer polls the
communicator's abort word and takes its budget from ``MINI_NCCL_WATCHDOG_TIMEOUT_MS``, the watchdog
times the kernel like a collective, and a wait that gives up fails the communicator for good
(``Communicator.async_error()``; every later call raises).
"""
from __future__ import annotations

import ctypes as C
import os

from .._lib import lib

BM = 128


def _native():
    L = lib()
    if not hasattr(L, "mncclGemmReduceScatterBf16"):
        raise RuntimeError("libmini_nccl.so was built without the fused GEMM kernels (csrc/kernels/gemm_fused.cu)")
    return L


def _sym(comm, numel, dtype):
    import torch

    if comm.size > 1:
        t = comm.empty(numel, dtype)
    else:
        t = torch.empty(numel, dtype=dtype, device="cuda")
    t.zero_()
    return t


def _check_comm(comm):
    """A communicator that has failed (watchdog trip, a kernel's failed wait, abort) takes no more work."""
    err = comm.async_error()
    if err != 0:
        from .._lib import MiniNcclError

        raise MiniNcclError(err, "fused kernel on a failed communicator")


def _peers(comm, tensor):
    if comm.size == 1:
        return (C.c_void_p * 1)(tensor.data_ptr())
    ptrs, _ = comm.peer_pointers(tensor)
    return (C.c_void_p * comm.size)(*ptrs)


class GemmReduceScatter:
    def __init__(self, comm, M: int, N: int):
        import torch

        L = _native()
        R = comm.size
        if M % R or (M // R) % BM or N % 8:
            raise ValueError("M / ranks must be a multiple of 128 and N a multiple of 8")
        self.comm, self.M, self.N = comm, M, N
        self.stage = _sym(comm, L.mncclGemmRsStageBytes(M, N, R), torch.uint8)
        self.flags = _sym(comm, max(4, L.mncclGemmRsFlagWords(M, N, R)), torch.int32)
        self.state = torch.zeros(4, dtype=torch.int32, device="cuda")
        torch.cuda.synchronize()
        if R > 1:
            comm.barrier()
        self._stage_peers = _peers(comm, self.stage)
        self._flag_peers = _peers(comm, self.flags)
        self._handle = comm.device_handle_bytes()
        # multicast address of the staging: the in-switch sum needs it (0: peer-to-peer kernel).  The
        # in-switch form is the default on up to four ranks, where it has been measured (TP=4: 116.8
        # against 121.4 us); with more ranks it has to be asked for (MINI_NCCL_RS_SWITCH=1).
        self._mc = 0
        want = os.environ.get("MINI_NCCL_RS_SWITCH", "1" if R <= 4 else "0")
        if R > 1 and want != "0" and hasattr(L, "mncclGemmReduceScatterBf16Switch"):
            self._mc = comm.peer_pointers(self.stage)[1]
        # CTAs that only sum finished tiles in the switch form (0: the kernel's default of 16)
        self.n_comm_ctas = int(os.environ.get("MINI_NCCL_RS_COMM_CTAS", "0"))

    @property
    def in_switch(self) -> bool:
        """True when the sum of the partial tiles is taken by the NVSwitch."""
        return self._mc != 0

    def __call__(self, a, b, out=None, stream=None):
        """``a [M, K_r]``, ``b [N, K_r]`` bf16 -> ``out [M / ranks, N]`` bf16 (this rank's rows of the sum)."""
        import torch

        M, N = self.M, self.N
        if tuple(a.shape)[0] != M or tuple(b.shape)[0] != N or a.shape[1] != b.shape[1]:
            raise ValueError("shape mismatch")
        if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16 or a.stride(1) != 1 or b.stride(1) != 1:
            raise TypeError("bf16 operands with a unit inner stride")
        if out is None:
            out = torch.empty((M // self.comm.size, N), dtype=torch.bfloat16, device=a.device)
        s = stream.cuda_stream if stream is not None else torch.cuda.current_stream().cuda_stream
        _check_comm(self.comm)
        if self._mc and out.stride(0) % 8 == 0 and out.data_ptr() % 16 == 0:
            rc = _native().mncclGemmReduceScatterBf16Switch(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, a.shape[1],
                                                            a.stride(0), b.stride(0), out.stride(0), self.comm.rank,
                                                            self.comm.size, self._stage_peers, self._flag_peers,
                                                            self.state.data_ptr(), self._mc, self.n_comm_ctas,
                                                            self._handle, len(self._handle), s)
        else:
            rc = _native().mncclGemmReduceScatterBf16Comm(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, a.shape[1],
                                                          a.stride(0), b.stride(0), out.stride(0), self.comm.rank,
                                                          self.comm.size, self._stage_peers, self._flag_peers,
                                                          self.state.data_ptr(), self._handle, len(self._handle), s)
        if rc != 0:
            raise RuntimeError(f"mncclGemmReduceScatterBf16 failed with code {rc}")
        return out


class AllGatherGemm:
    def __init__(self, comm, M: int, K: int, n_comm_ctas: int = 0):
        import torch

        L = _native()
        R = comm.size
        if M % R or (M // R) % BM or K % 8:
            raise ValueError("M / ranks must be a multiple of 128 and K a multiple of 8")
        self.comm, self.M, self.K, self.n_comm = comm, M, K, n_comm_ctas
        self.gather = _sym(comm, M * K, torch.bfloat16).view(M, K)   # X of every rank lands here
        self.ready = _sym(comm, max(4, L.mncclAgGemmReadyWords(M)), torch.int32)
        self.bar = _sym(comm, max(4, L.mncclAgGemmBarWords(R, max(n_comm_ctas, 74))), torch.int32)
        self.state = torch.zeros(4, dtype=torch.int32, device="cuda")
        torch.cuda.synchronize()
        if R > 1:
            comm.barrier()
        self._xg = _peers(comm, self.gather)
        self._ready = _peers(comm, self.ready)
        self._bar = _peers(comm, self.bar)
        self._handle = comm.device_handle_bytes()

    @property
    def local_shard(self):
        """The rows of the gather buffer this rank fills before calling (write the input here)."""
        r, per = self.comm.rank, self.M // self.comm.size
        return self.gather[r * per:(r + 1) * per]

    def __call__(self, b, out=None, stream=None, swiglu: bool = False):
        """``b [N_r, K]`` bf16 -> ``out [M, N_r]`` bf16 = (all ranks' shards stacked) @ b.T.

        ``swiglu=True``: the epilogue applies SwiGLU and ``out`` is ``[M, N_r / 2]``; the rows of ``b`` must then
        be interleaved in groups of 16 (:func:`interleave_gate_up`), N_r a multiple of 32."""
        import torch

        if b.dtype != torch.bfloat16 or b.shape[1] != self.K or b.stride(1) != 1:
            raise TypeError("b must be bf16 [N, K] with a unit inner stride")
        N = b.shape[0]
        if swiglu and N % 32:
            raise ValueError("SwiGLU in the epilogue needs N a multiple of 32")
        n_out = N // 2 if swiglu else N
        if out is None:
            out = torch.empty((self.M, n_out), dtype=torch.bfloat16, device=b.device)
        if tuple(out.shape) != (self.M, n_out) or out.dtype != torch.bfloat16 or out.stride(1) != 1:
            raise ValueError(f"out must be bf16 [{self.M}, {n_out}] with a unit inner stride")
        s = stream.cuda_stream if stream is not None else torch.cuda.current_stream().cuda_stream
        _check_comm(self.comm)
        rc = _native().mncclAllGatherGemmBf16Comm(self._xg, b.data_ptr(), out.data_ptr(), self.M, N, self.K, self.K, b.stride(0),
                                                  out.stride(0), self.comm.rank, self.comm.size, self._ready, self._bar,
                                                  self.state.data_ptr(), self.n_comm, 1 if swiglu else 0, self._handle,
                                                  len(self._handle), s)
        if rc != 0:
            raise RuntimeError(f"all-gather->GEMM kernel failed with code {rc}")
        return out


def interleave_gate_up(w_gate, w_up):
    """Weight layout for SwiGLU in the all-gather->GEMM epilogue: ``[2F, K]`` whose rows alternate between 16 gate
    features and the 16 up features of the same indices, so that one 32-column piece of an accumulator row holds
    both operands of 16 outputs.  ``F`` must be a multiple of 16."""
    import torch

    F, K = w_gate.shape
    if tuple(w_up.shape) != (F, K) or F % 16:
        raise ValueError("gate and up must both be [F, K] with F a multiple of 16")
    return torch.stack((w_gate.reshape(F // 16, 16, K), w_up.reshape(F // 16, 16, K)), dim=1).reshape(2 * F, K).contiguous()


def split_gate_up(h):
    """Inverse view for a product with interleaved weights: ``h [M, 2F]`` -> ``(gate [M, F], up [M, F])``."""
    M, N = h.shape
    v = h.reshape(M, N // 32, 2, 16)
    return v[:, :, 0, :].reshape(M, N // 2), v[:, :, 1, :].reshape(M, N // 2)
