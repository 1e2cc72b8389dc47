"""Interop helpers between raw device pointers and torch tensors."""
from __future__ import annotations


def tensor_from_ptr(ptr: int, nbytes: int, dtype=None, device=None, owner=None):
    """A torch tensor viewing ``nbytes`` of device memory at ``ptr`` (no copy, no ownership).

    ``owner`` is kept alive by the tensor's holder object."""
    import torch

    class _Holder:
        pass

    h = _Holder()
    h.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (int(ptr), False), "version": 3}
    h.owner = owner
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    raw = torch.as_tensor(h, device=dev)
    return raw if dtype is None else raw.view(dtype)
