"""Communicator: the thin PyTorch-facing wrapper around the C ABI.

Tensors are passed by data pointer; the collective is enqueued on the current
CUDA stream (or on the stream given) and returns immediately.  Buffers from
:meth:`Communicator.empty` live in symmetric memory (mapped into every peer and
bound to the NVSwitch multicast object when NVLS is available), so collectives
on them are zero-copy.  The reference has no Python layer; its C ABI
(reference: include/mini_nccl_api.h:55-69) is what this wraps.
"""
from __future__ import annotations

import ctypes as C
import json
import os
from typing import Optional, Sequence

from . import _lib
from ._lib import MiniNcclError, check, lib

try:  # torch is only needed for the tensor helpers
    import torch
except Exception:  # pragma: no cover
    torch = None


_DTYPE_TABLE: dict = {}


def _torch_dtype_code(dt) -> int:
    code = _DTYPE_TABLE.get(dt)
    if code is not None:
        return code
    table = {
        torch.int8: _lib.INT8, torch.uint8: _lib.UINT8, torch.int32: _lib.INT32, torch.int64: _lib.INT64,
        torch.float16: _lib.FLOAT16, torch.float32: _lib.FLOAT32, torch.float64: _lib.FLOAT64,
        torch.bfloat16: _lib.BFLOAT16,
    }
    for name, code in (("uint32", _lib.UINT32), ("uint64", _lib.UINT64)):
        if hasattr(torch, name):
            table[getattr(torch, name)] = code
    if dt not in table:
        raise TypeError(f"unsupported dtype {dt}")
    _DTYPE_TABLE.update(table)
    return table[dt]


_OPS = {"sum": _lib.SUM, "prod": _lib.PROD, "max": _lib.MAX, "min": _lib.MIN, "avg": _lib.AVG}
_ALGOS = {"auto": 0, "ll": 1, "oneshot": 2, "twoshot": 3, "nvls": 4, "ring": 5, "pipe": 7}


class Communicator:
    """One rank's handle.  ``rank=-1`` asks the Hera master at ``ip`` for a rank."""

    def __init__(self, nranks: int, rank: int, ip: str = "127.0.0.1"):
        self._h = C.c_void_p()
        self._symmetric = {}  # data_ptr -> (nbytes, keepalive)
        check(lib().mncclCommInitRank(C.byref(self._h), nranks, rank, ip.encode()), "mncclCommInitRank")
        r, n = C.c_int(), C.c_int()
        check(lib().mncclCommUserRank(self._h, C.byref(r)), "mncclCommUserRank")
        check(lib().mncclCommCount(self._h, C.byref(n)), "mncclCommCount")
        self.rank, self.size = r.value, n.value

    @classmethod
    def from_env(cls) -> "Communicator":
        """RANK / WORLD_SIZE / MASTER_ADDR as torchrun sets them.  The bootstrap port is
        MINI_NCCL_BOOTSTRAP_PORT (default 8888), independent of MASTER_PORT."""
        rank = int(os.environ.get("RANK", "0"))
        world = int(os.environ.get("WORLD_SIZE", "1"))
        return cls(world, rank, os.environ.get("MASTER_ADDR", "127.0.0.1"))

    # ------------------------------------------------------------------ lifecycle
    def destroy(self) -> None:
        if self._h:
            h, self._h = self._h, C.c_void_p()
            self._symmetric.clear()
            check(lib().mncclCommDestroy(h), "mncclCommDestroy")

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass

    @property
    def handle(self) -> C.c_void_p:
        return self._h

    # ------------------------------------------------------------------ collectives
    @staticmethod
    def _stream_ptr(stream) -> int:
        if stream is None:
            if torch is not None and torch.cuda.is_available():
                return torch.cuda.current_stream().cuda_stream
            return 0
        return stream.cuda_stream if hasattr(stream, "cuda_stream") else int(stream)

    def all_reduce(self, tensor, op: str = "sum", out=None, scale: float = 1.0, wire_dtype=None,
                   algo: str = "auto", stream=None):
        """``out = scale * reduce(tensor)`` over all ranks (in place when ``out`` is None).

        ``out`` may have another floating dtype than ``tensor`` and ``wire_dtype`` may name the
        type the data crosses NVLink in (fp32 -> bf16 -> fp32 and the like); accumulation is
        always fp32."""
        out = tensor if out is None else out
        if not tensor.is_contiguous() or not out.is_contiguous():
            raise ValueError("all_reduce needs contiguous tensors")
        if out.numel() != tensor.numel():
            raise ValueError("size mismatch")
        st = _torch_dtype_code(tensor.dtype)
        rt = _torch_dtype_code(out.dtype)
        wt = _torch_dtype_code(wire_dtype) if wire_dtype is not None else (rt if st == rt else _lib.BFLOAT16)
        check(lib().mncclAllReduceEx(tensor.data_ptr(), st, out.data_ptr(), rt, wt, tensor.numel(), _OPS[op],
                                     float(scale), _ALGOS[algo], self._h, self._stream_ptr(stream)), "mncclAllReduceEx")
        return out

    def reduce_scatter(self, tensor, out, op: str = "sum", stream=None):
        if tensor.numel() != out.numel() * self.size:
            raise ValueError("reduce_scatter: input must hold size * out.numel() elements")
        check(lib().mncclReduceScatter(tensor.data_ptr(), out.data_ptr(), out.numel(), _torch_dtype_code(tensor.dtype),
                                       _OPS[op], self._h, self._stream_ptr(stream)), "mncclReduceScatter")
        return out

    def all_gather(self, tensor, out, stream=None):
        if out.numel() != tensor.numel() * self.size:
            raise ValueError("all_gather: output must hold size * tensor.numel() elements")
        check(lib().mncclAllGather(tensor.data_ptr(), out.data_ptr(), tensor.numel(), _torch_dtype_code(tensor.dtype),
                                   self._h, self._stream_ptr(stream)), "mncclAllGather")
        return out

    def all_reduce_raw(self, send_ptr: int, recv_ptr: int, count: int, dtype: int, op: int = _lib.SUM, stream: int = 0):
        check(lib().mncclAllReduce(send_ptr, recv_ptr, count, dtype, op, self._h, stream), "mncclAllReduce")

    # ------------------------------------------------------------------ symmetric memory
    def empty(self, shape: Sequence[int] | int, dtype=None, device=None):
        """A tensor in symmetric memory.  Collective: every rank, same order, same size."""
        dtype = dtype or torch.float32
        if isinstance(shape, int):
            shape = (shape,)
        numel = 1
        for s in shape:
            numel *= int(s)
        nbytes = max(numel * torch.empty((), dtype=dtype).element_size(), 16)
        ptr = C.c_void_p()
        check(lib().mncclMemAlloc(self._h, nbytes, C.byref(ptr)), "mncclMemAlloc")
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)

        class _Holder:  # exposes the allocation through __cuda_array_interface__
            pass

        h = _Holder()
        h.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr.value, False), "version": 3}
        raw = torch.as_tensor(h, device=dev)
        t = raw.view(dtype)[:numel].view(*shape)
        self._symmetric[ptr.value] = (nbytes, h)
        return t

    def free(self, tensor) -> None:
        """Collective counterpart of :meth:`empty`."""
        ptr = tensor.data_ptr()
        if ptr not in self._symmetric:
            raise ValueError("tensor was not allocated by Communicator.empty")
        del self._symmetric[ptr]
        check(lib().mncclMemFree(self._h, ptr), "mncclMemFree")

    def register(self, tensor) -> None:
        """Collective: exchange CUDA IPC handles for an ordinary device tensor so that the peer-to-peer
        algorithms use it in place.  Same size on every rank."""
        check(lib().mncclCommRegister(self._h, tensor.data_ptr(), tensor.numel() * tensor.element_size()), "mncclCommRegister")

    def deregister(self, tensor) -> None:
        check(lib().mncclCommDeregister(self._h, tensor.data_ptr()), "mncclCommDeregister")

    def peer_pointers(self, tensor):
        peers = (C.c_void_p * self.size)()
        mc = C.c_void_p()
        check(lib().mncclMemPeerPointers(self._h, tensor.data_ptr(), peers, C.byref(mc)), "mncclMemPeerPointers")
        return [p or 0 for p in peers], (mc.value or 0)

    # ------------------------------------------------------------------ control
    def barrier(self) -> None:
        check(lib().mncclBarrier(self._h), "mncclBarrier")

    def abort(self) -> None:
        check(lib().mncclCommAbort(self._h), "mncclCommAbort")

    def async_error(self) -> int:
        e = C.c_int()
        check(lib().mncclCommGetAsyncError(self._h, C.byref(e)), "mncclCommGetAsyncError")
        return e.value

    def stats(self) -> dict:
        buf = C.create_string_buffer(4096)
        check(lib().mncclCommStats(self._h, buf, len(buf)), "mncclCommStats")
        return json.loads(buf.value.decode())

    def set_tuning(self, max_blocks: int = 0, unroll: int = 0) -> None:
        """Grid cap and NVLS unroll for the calls that follow (0 = built-in).  Same values on every rank."""
        check(lib().mncclCommSetTuning(self._h, max_blocks, unroll), "mncclCommSetTuning")

    def set_knob(self, name: str, value: int) -> None:
        """One launch-tuning knob by the name of its environment variable without the ``MINI_NCCL_``
        prefix (``"PIPE_CHUNK_BYTES"``, ``"NVLS_P2P_PERMILLE"``, ...).  Same value on every rank."""
        check(lib().mncclCommSetKnob(self._h, name.encode(), int(value)), "mncclCommSetKnob(%s)" % name)

    def query_algo(self, nbytes: int, dtype=None, op: str = "sum", registered: bool = False) -> str:
        a = C.c_int()
        code = _torch_dtype_code(dtype) if dtype is not None else _lib.FLOAT32
        check(lib().mncclCommQueryAlgo(self._h, nbytes, code, _OPS[op], int(registered), C.byref(a)), "mncclCommQueryAlgo")
        return _lib.ALGO_NAMES.get(a.value, "?")

    def device_handle_bytes(self) -> bytes:
        need = C.c_size_t()
        check(lib().mncclCommDeviceHandle(self._h, None, 0, C.byref(need)), "mncclCommDeviceHandle")
        buf = C.create_string_buffer(need.value)
        check(lib().mncclCommDeviceHandle(self._h, buf, need.value, None), "mncclCommDeviceHandle")
        return buf.raw
