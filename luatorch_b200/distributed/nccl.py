"""`lf.distributed.nccl`: allreduce / broadcast over the job's ranks
(lua/luatorch/distributed/nccl.lua:13-51).

The reference functions take one tensor PER GPU because a single process drives every
device.  With one rank per GPU each rank passes its own tensor (or a list of its tensors):
`allreduce` averages in place across ranks, `broadcast` copies the root rank's values.  A
one-entry-per-rank list (the reference's calling convention) is accepted when the world is a
single process: its entries are averaged among themselves.
"""
from __future__ import annotations

from typing import Sequence, Union

import torch

from ..tensor import Tensor
from . import comm

_staging = {}


def _stage(nbytes: int):
    if not (torch.cuda.is_available() and comm.world_size() > 1):
        return None
    size = max(1 << 22, 1 << (int(nbytes) - 1).bit_length())
    buf = _staging.get(size)
    if buf is None:
        buf = comm.SymmetricBuffer(size)
        _staging[size] = buf
    return buf if buf.peer_mapped else None


def allreduce(tensors: Union[Tensor, Sequence[Tensor]]) -> bool:
    single = isinstance(tensors, Tensor)
    items = [tensors] if single else list(tensors)
    if comm.world_size() == 1:
        if len(items) > 1 and all(t.numel() == items[0].numel() for t in items):
            mean = sum(t._t.float() for t in items) / len(items)
            for t in items:
                t._t.copy_(mean.to(t._t.dtype))
        return True
    for t in items:
        x = t._t if t._t.is_contiguous() else t._t.contiguous()
        comm.allreduce_mean_(x, _stage(x.numel() * x.element_size() + 256))
        if x is not t._t:
            t._t.copy_(x)
    return True


def broadcast(tensors: Union[Tensor, Sequence[Tensor]], root: int = 0, num_gpus: int = None) -> bool:
    single = isinstance(tensors, Tensor)
    items = [tensors] if single else list(tensors)
    if comm.world_size() == 1:
        if len(items) > 1:
            for t in items:
                if t is not items[root]:
                    t._t.copy_(items[root]._t)
        return True
    for t in items:
        x = t._t if t._t.is_contiguous() else t._t.contiguous()
        comm.broadcast_(x, root, _stage(x.numel() * x.element_size()))
        if x is not t._t:
            t._t.copy_(x)
    return True
