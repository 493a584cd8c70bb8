"""Flat parameter arenas: every parameter of a model becomes a view into

    master   fp32   the weights the optimizer updates (what checkpoints save)
    shadow   bf16   the copy the forward / backward kernels read
    grad     bf16   where the backward kernels write gradients, in place

laid out in `parameters()` order, each storage unit padded to 256 elements, the whole arena
padded so any bucket can be cut at a multiple of 2048 elements.  One launch can then update
the whole model (the reference launches one Adam kernel per tensor,
lua/luatorch/optim/adam.lua:44-86) and a gradient bucket is a contiguous byte range that the
fused all-reduce kernels address on every rank with the same offset.

Storage units: a parameter that is a column slice of a fused tensor (attention q/k/v) is
stored through its base; the slices stay views of it.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence

import torch

from .. import _backend as B
from ..tensor import Tensor

ALIGN = 256          # elements per storage-unit granule
BUCKET_ALIGN = 2048  # bucket boundaries (multiple of 8 * 16 ranks * ...) in elements

_ARENAS: Dict[int, "ParamArena"] = {}


def arena_of(p: Tensor) -> Optional["ParamArena"]:
    return _ARENAS.get(id(p))


def storage_units(params: Sequence[Tensor]) -> List[Tensor]:
    """Unique storage tensors behind `params`, in first-seen order."""
    seen, units = set(), []
    for p in params:
        u = p._base if p._base is not None else p
        if id(u) not in seen:
            seen.add(id(u))
            units.append(u)
    return units


class ParamArena:
    def __init__(self, params: Sequence[Tensor], device: str = "cuda",
                 compute_dtype: Optional[torch.dtype] = torch.bfloat16,
                 grad_dtype: torch.dtype = torch.bfloat16,
                 allocator: Optional[Callable[[int, torch.dtype], torch.Tensor]] = None):
        self.params = list(params)
        self.units = storage_units(self.params)
        self.device = torch.device(device)
        self.offsets: List[int] = []
        off = 0
        for u in self.units:
            self.offsets.append(off)
            off += (u.numel() + ALIGN - 1) // ALIGN * ALIGN
        self.used = off
        self.total = (off + BUCKET_ALIGN - 1) // BUCKET_ALIGN * BUCKET_ALIGN
        alloc = allocator or (lambda n, dt: torch.zeros(n, device=self.device, dtype=dt))
        self.master = torch.zeros(self.total, device=self.device, dtype=torch.float32)
        self.shadow = alloc(self.total, compute_dtype) if compute_dtype is not None else None
        self.grad = alloc(self.total, grad_dtype)
        self.compute_dtype = compute_dtype
        self.grad_dtype = grad_dtype
        for u, o in zip(self.units, self.offsets):
            n = u.numel()
            shape = list(u._t.shape)
            self.master[o:o + n].copy_(u._t.reshape(-1).to(self.device, torch.float32))
            u._t = self.master[o:o + n].view(shape)
            u._grad_buf = self.grad[o:o + n].view(shape)
            u._compute = self.shadow[o:o + n].view(shape) if self.shadow is not None else None
            u.grad = None
            _ARENAS[id(u)] = self
        for p in self.params:
            if p._base is not None:
                lo, hi = p._base_slice
                base = p._base
                p._t = base._t[:, lo:hi]
                p._grad_buf = base._grad_buf[:, lo:hi]
                p._compute = base._compute[:, lo:hi] if base._compute is not None else None
                p.grad = None
            _ARENAS[id(p)] = self
        self.sync_shadow()

    # ------------------------------------------------------------------ views / bookkeeping
    def unit_range(self, u: Tensor):
        i = next(k for k, x in enumerate(self.units) if x is u)
        return self.offsets[i], self.offsets[i] + u.numel()

    def sync_shadow(self) -> None:
        """shadow <- master (after loading a checkpoint or editing master by hand)."""
        if self.shadow is None:
            return
        if self.master.is_cuda:
            B.ext().cast_into(self.master, self.shadow)
        else:
            self.shadow.copy_(self.master)

    def zero_grad(self) -> None:
        for p in self.params:
            p.grad = None
        for u in self.units:
            u.grad = None

    def segments(self, decay_of: Callable[[Tensor], float]):
        """(seg_end int64[n], seg_wd fp32[n]) device tensors in arena coordinates; adjacent
        units with equal decay are merged."""
        ends, wds = [], []
        for i, u in enumerate(self.units):
            end = self.offsets[i + 1] if i + 1 < len(self.units) else self.total
            wd = float(decay_of(u))
            if wds and wds[-1] == wd:
                ends[-1] = end
            else:
                ends.append(end)
                wds.append(wd)
        return (torch.tensor(ends, device=self.device, dtype=torch.int64),
                torch.tensor(wds, device=self.device, dtype=torch.float32))

    def buckets(self, bucket_elems: int):
        """Contiguous [start, end) element ranges cut near unit boundaries (rounded down to
        BUCKET_ALIGN), listed from the END of the arena (the order gradients become ready in
        backward).  `units` lists every storage unit overlapping the range: the bucket may be
        reduced once all of them have their final gradient."""
        bounds = [self.total]
        cur_end = self.total
        for i in range(len(self.units) - 1, -1, -1):
            start = self.offsets[i] // BUCKET_ALIGN * BUCKET_ALIGN
            if cur_end - start >= bucket_elems and start < bounds[-1]:
                bounds.append(start)
                cur_end = start
        if bounds[-1] != 0:
            bounds.append(0)
        out = []
        for hi, lo in zip(bounds[:-1], bounds[1:]):
            members = [u for u, o in zip(self.units, self.offsets)
                       if o < hi and o + u.numel() > lo]
            out.append({"start": lo, "end": hi, "units": members})
        return out
