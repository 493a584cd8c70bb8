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
BUCKET_ALIGN = 2048  # bucket boundaries in elements: a multiple of 8 * world for worlds 2, 4, 8, 16


def bucket_align_for(world: int) -> int:
    """Bucket boundaries must be multiples of 8 * world (16-byte vectors, one slice per rank):
    2048 for power-of-two worlds, lcm(2048, 8 * world) otherwise (3, 5, 6, 7 ranks)."""
    import math
    w = max(1, int(world))
    return BUCKET_ALIGN * (8 * w) // math.gcd(BUCKET_ALIGN, 8 * w)


class StateShards:
    """Memory-sharded optimizer state: of every bucket [start, end) rank r keeps slice r, and
    the slices of all buckets sit back to back in one compact tensor per state array (fp32
    master, m, v), `numel` = arena size / world elements long.  `pieces[i]` = (start, span,
    shard_offset) of bucket i.  The reference keeps full state on its one device
    (lua/luatorch/optim/adamw.lua:19-49)."""

    def __init__(self, buckets, rank: int, world: int):
        self.rank, self.world = int(rank), int(world)
        self.pieces = []
        off = 0
        for b in buckets:
            span = (b["end"] - b["start"]) // self.world
            assert span * self.world == b["end"] - b["start"], "bucket not divisible by the world size"
            self.pieces.append((b["start"], span, off))
            off += span
        self.numel = off

    def take(self, full: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """This rank's slices of a full-length arena tensor, compacted."""
        if out is None:
            out = torch.empty(self.numel, device=full.device, dtype=full.dtype)
        for start, span, off in self.pieces:
            lo = start + self.rank * span
            out[off:off + span].copy_(full[lo:lo + span])
        return out

    def gather(self, shard: torch.Tensor, total: int) -> torch.Tensor:
        """Full-length tensor assembled from every rank's shard (collective: all ranks call)."""
        import torch.distributed as dist
        full = torch.zeros(total, device=shard.device, dtype=shard.dtype)
        for start, span, off in self.pieces:
            if span == 0:
                continue
            dist.all_gather_into_tensor(full[start:start + span * self.world],
                                        shard[off:off + span].contiguous())
        return full

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
                 allocator: Optional[Callable[[int, torch.dtype], torch.Tensor]] = None,
                 bucket_align: int = BUCKET_ALIGN):
        self.params = list(params)
        self.bucket_align = int(bucket_align)
        self.state_shards: Optional[StateShards] = None
        self.master_shard: Optional[torch.Tensor] = None
        self.units = storage_units(self.params)
        self.device = torch.device(device)
        self.offsets: List[int] = []
        off = 0
        for u in self.units:
            self.offsets.append(off)
            off += (u.numel() + ALIGN - 1) // ALIGN * ALIGN
        self.used = off
        self.total = (off + self.bucket_align - 1) // self.bucket_align * self.bucket_align
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
            u._grad_buf = self.grad[o:o + n].view(shape)
            u._compute = self.shadow[o:o + n].view(shape) if self.shadow is not None else None
            u.grad = None
            _ARENAS[id(u)] = self
        for p in self.params:
            if p._base is not None:
                lo, hi = p._base_slice
                base = p._base
                p._grad_buf = base._grad_buf[:, lo:hi]
                p._compute = base._compute[:, lo:hi] if base._compute is not None else None
                p.grad = None
            _ARENAS[id(p)] = self
        self._point_values(self.master)
        self.sync_shadow()

    def _point_values(self, flat: torch.Tensor) -> None:
        """Make every parameter's value tensor (`_t`) a view of the flat tensor `flat`."""
        for u, o in zip(self.units, self.offsets):
            u._t = flat[o:o + u.numel()].view(list(u._grad_buf.shape))
        for p in self.params:
            if p._base is not None:
                lo, hi = p._base_slice
                p._t = p._base._t[:, lo:hi]

    # ------------------------------------------------------------------ sharded optimizer state
    def state_numel(self) -> int:
        """Length of one optimizer-state array on this rank."""
        return self.state_shards.numel if self.state_shards is not None else self.total

    def shard_state(self, shards: StateShards) -> None:
        """Keep only this rank's slices of the fp32 master (and let optimizers built afterwards
        allocate their moments at shard size).  Parameter values then read from the bf16
        shadow until `materialize_master()` assembles the full fp32 copy again."""
        assert self.shadow is not None and self.master is not None
        self.state_shards = shards
        self.master_shard = shards.take(self.master)
        self.master = None
        self._point_values(self.shadow)

    def materialize_master(self) -> None:
        """Collective.  Assemble the full fp32 master from every rank's shard (before writing a
        checkpoint or loading one); parameter values are views of it until release_master()."""
        if self.state_shards is None or self.master is not None:
            return
        self.master = self.state_shards.gather(self.master_shard, self.total)
        self._point_values(self.master)

    def release_master(self, write_back: bool = False) -> None:
        """Drop the assembled master again; with `write_back` its values first replace this
        rank's shard and the bf16 shadow (after loading a checkpoint into it)."""
        if self.state_shards is None or self.master is None:
            return
        if write_back:
            self.state_shards.take(self.master, out=self.master_shard)
            self.sync_shadow()
        self.master = None
        self._point_values(self.shadow)

    # ------------------------------------------------------------------ views / bookkeeping
    def unit_range(self, u: Tensor):
        i = next(k for k, x in enumerate(self.units) if x is u)
        return self.offsets[i], self.offsets[i] + u.numel()

    def sync_shadow(self) -> None:
        """shadow <- master (after loading a checkpoint or editing master by hand)."""
        if self.shadow is None or self.master is None:
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
            start = self.offsets[i] // self.bucket_align * self.bucket_align
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
