"""Data parallelism on top of the communicator.

The reference stops at the AllReduce call; there is no training integration.
Here gradients are packed into flat buckets of ~25 MB that live in symmetric
memory, parameters' ``.grad`` are views into them (no gather copy), and each
bucket is reduced as soon as its last gradient has been accumulated, on a side
stream, so communication overlaps the rest of the backward pass.  The AllReduce
is fused with the 1/world scale and, optionally, with a cast to an fp32
main-gradient buffer (bf16 on the wire, fp32 accumulation, fp32 result), all in
the one communication kernel.

A stock training loop may rebind ``param.grad`` (``optimizer.zero_grad()`` sets it to ``None`` by
default, after which autograd allocates a fresh tensor): the gradient hook notices, copies such a
gradient into its bucket slot and points ``param.grad`` back at the slot, so the bucket that is
reduced always holds the step's gradients.  ``no_sync()`` skips the reduction for gradient
accumulation; accumulating WITHOUT it is also correct (the already averaged part is the same on
every rank, so averaging it again changes nothing), just one collective per micro-step.

``allreduce_comm_hook`` is the same reduction packaged for
``torch.nn.parallel.DistributedDataParallel.register_comm_hook``.
"""
from __future__ import annotations

import contextlib
from typing import Optional

import torch
import torch.nn as nn


class _Bucket:
    __slots__ = ("flat", "main", "params", "pending", "reduced", "index")

    def __init__(self, index):
        self.index = index
        self.flat = None      # gradient bucket (param dtype), symmetric memory when world > 1
        self.main = None      # optional fp32 main-gradient bucket
        self.params = []
        self.pending = 0
        self.reduced = False


class DistributedDataParallel(nn.Module):
    """Bucketed, overlapped gradient AllReduce through mini_nccl_b200.

    Args:
      module: the model (already on the GPU).
      comm: a Communicator.
      bucket_mb: bucket capacity in MB (25 as in the benchmark configuration).
      main_grad_dtype: when set (torch.float32), every bucket has a second buffer of that
        type that receives ``sum(grads) / world`` (fused cast); ``param.main_grad`` views it.
      overlap: reduce buckets on a side stream during backward (True) or after it (False).
    """

    def __init__(self, module: nn.Module, comm, bucket_mb: float = 25.0, main_grad_dtype: Optional[torch.dtype] = None,
                 overlap: bool = True):
        super().__init__()
        self.module = module
        self.comm = comm
        self.world = comm.size
        self.overlap = overlap
        self.main_grad_dtype = main_grad_dtype
        self.comm_stream = torch.cuda.Stream()
        self._buckets: list[_Bucket] = []
        self._param_bucket = {}
        self._callback_queued = False
        self._sync = True
        self._slot = {}          # id(param) -> its view into the bucket
        self.launches = 0
        self.repaired = 0        # gradients found outside their bucket and moved back in
        self._build_buckets(int(bucket_mb * 1024 * 1024))
        self._broadcast_parameters()
        for p in self._params():
            p.register_post_accumulate_grad_hook(self._on_grad)

    # -------------------------------------------------------------- construction
    def _params(self):
        seen = set()
        for p in self.module.parameters():
            if p.requires_grad and id(p) not in seen:
                seen.add(id(p))
                yield p

    def _build_buckets(self, cap_bytes: int):
        # Reverse registration order approximates the order gradients become ready.
        groups, cur, cur_bytes, cur_dtype = [], [], 0, None
        for p in reversed(list(self._params())):
            nbytes = p.numel() * p.element_size()
            if cur and (cur_bytes + nbytes > cap_bytes or p.dtype != cur_dtype):
                groups.append(cur)
                cur, cur_bytes = [], 0
            cur.append(p)
            cur_bytes += nbytes
            cur_dtype = p.dtype
        if cur:
            groups.append(cur)
        for i, params in enumerate(groups):
            b = _Bucket(i)
            # 16-byte aligned slots so that every view keeps vector alignment
            align = 16 // params[0].element_size()
            offsets, total = [], 0
            for p in params:
                offsets.append(total)
                total += (p.numel() + align - 1) // align * align
            dtype = params[0].dtype
            b.flat = self.comm.empty(total, dtype) if self.world > 1 else torch.empty(total, dtype=dtype, device="cuda")
            b.flat.zero_()
            if self.main_grad_dtype is not None:
                b.main = (self.comm.empty(total, self.main_grad_dtype) if self.world > 1
                          else torch.empty(total, dtype=self.main_grad_dtype, device="cuda"))
                b.main.zero_()
            for p, off in zip(params, offsets):
                p.grad = b.flat[off:off + p.numel()].view_as(p)
                self._slot[id(p)] = p.grad
                if b.main is not None:
                    p.main_grad = b.main[off:off + p.numel()].view_as(p)
                self._param_bucket[id(p)] = b
            b.params = params
            self._buckets.append(b)

    def _broadcast_parameters(self):
        # Same initial weights everywhere: AllReduce of (rank 0's value, zeros elsewhere).
        if self.world == 1:
            return
        for p in self._params():
            if self.comm.rank != 0:
                p.data.zero_()
            flat = p.data.view(-1)
            self.comm.all_reduce(flat, "sum")
        torch.cuda.synchronize()

    # -------------------------------------------------------------- backward hooks
    def _on_grad(self, p):
        b = self._param_bucket[id(p)]
        slot = self._slot[id(p)]
        if p.grad is not slot and (p.grad is None or p.grad.data_ptr() != slot.data_ptr()):
            # Someone rebound .grad (zero_grad(set_to_none=True), a manual assignment): the bucket slot holds
            # stale data.  Move the fresh gradient in and make .grad the view again.
            with torch.no_grad():
                if p.grad is None:
                    slot.zero_()
                else:
                    slot.copy_(p.grad)
            p.grad = slot
            self.repaired += 1
        if not self._sync:
            return
        if b.pending == 0:
            b.pending = len(b.params)
        b.pending -= 1
        if not self._callback_queued:
            self._callback_queued = True
            torch.autograd.Variable._execution_engine.queue_callback(self._finish_backward)
        if b.pending == 0 and self.overlap:
            self._reduce_bucket(b)

    def _reduce_bucket(self, b: _Bucket):
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream())
        self.comm_stream.wait_event(ev)
        with torch.cuda.stream(self.comm_stream):
            if b.main is not None:
                self.comm.all_reduce(b.flat, "sum", out=b.main, scale=1.0 / self.world, wire_dtype=b.flat.dtype,
                                     stream=self.comm_stream)
            else:
                self.comm.all_reduce(b.flat, "sum", scale=1.0 / self.world, stream=self.comm_stream)
        b.reduced = True
        self.launches += 1

    def _finish_backward(self):
        self._callback_queued = False
        # Buckets not reduced during backward (overlap off, or a parameter that received no
        # gradient this step) are reduced now, in bucket order, identically on every rank.
        for b in self._buckets:
            if not b.reduced:
                self._reduce_bucket(b)
        torch.cuda.current_stream().wait_stream(self.comm_stream)
        for b in self._buckets:
            b.pending = 0
            b.reduced = False

    # -------------------------------------------------------------- module API
    def forward(self, *args, **kwargs):
        return self.module(*args, **kwargs)

    @contextlib.contextmanager
    def no_sync(self):
        """Backward passes inside this context only accumulate into the buckets; the first backward after it
        reduces the accumulated gradients (gradient accumulation with one collective per optimizer step)."""
        old, self._sync = self._sync, False
        try:
            yield
        finally:
            self._sync = old

    def zero_grad(self, set_to_none: bool = False):
        """Zeroes the buckets and keeps every ``.grad`` a view into them, whatever ``set_to_none`` says
        (prefer this to ``optimizer.zero_grad()``, which costs a copy per parameter in the next backward)."""
        for b in self._buckets:
            b.flat.zero_()
        for p in self._params():
            slot = self._slot[id(p)]
            if p.grad is not slot:
                p.grad = slot

    @property
    def buckets(self):
        return self._buckets

    def bucket_bytes(self):
        return [b.flat.numel() * b.flat.element_size() for b in self._buckets]


def allreduce_comm_hook(comm):
    """A comm hook for torch's own DistributedDataParallel: reduces ``bucket.buffer()`` with this
    library (fused 1/world scale) on the current stream and returns a completed future."""

    def hook(state, bucket):
        buf = bucket.buffer()
        comm.all_reduce(buf, "sum", scale=1.0 / comm.size)
        fut = torch.futures.Future()
        fut.set_result(buf)
        return fut

    return hook
