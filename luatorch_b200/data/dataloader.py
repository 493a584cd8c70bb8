"""Mini-batch iterator (lua/luatorch/data/dataloader.lua): `DataLoader(data, targets,
batch_size=32, shuffle=True)`, `iter()` yields `(batch_data, batch_targets)`, the last batch
may be short, `num_batches()`.

Batches are gathered with one indexed copy instead of per-element get/set; optional
extensions used by the data-parallel entry points: `rank` / `world_size` give every rank a
disjoint strided shard of each epoch's permutation, and `pin=True` stages batches in pinned
host memory so `Tensor.cuda_async()` overlaps the copy with compute."""
from __future__ import annotations

import math
from typing import Iterator, Tuple

import torch

from .. import _backend as B
from ..tensor import Tensor


class DataLoader:
    @classmethod
    def new(cls, *args, **kwargs):
        """`X.new(...)` is `X(...)`, the reference's constructor spelling."""
        return cls(*args, **kwargs)

    def __init__(self, data: Tensor, targets: Tensor, batch_size: int = 32, shuffle: bool = True,
                 rank: int = 0, world_size: int = 1, pin: bool = False):
        self.data = data
        self.targets = targets
        self.batch_size = batch_size or 32
        self.shuffle = shuffle is not False
        self.n_samples = data.shape[0]
        self.rank, self.world_size = rank, world_size
        self.pin = pin and torch.cuda.is_available()
        self.indices = torch.arange(self.n_samples)

    def _local_count(self) -> int:
        return len(range(self.rank, self.n_samples, self.world_size))

    def num_batches(self) -> int:
        return math.ceil(self._local_count() / self.batch_size)

    def iter(self) -> Iterator[Tuple[Tensor, Tensor]]:
        if self.shuffle:
            self.indices = torch.randperm(self.n_samples, generator=B.cpu_generator())
        idx = self.indices[self.rank::self.world_size]
        d, t = self.data._t, self.targets._t
        for pos in range(0, idx.numel(), self.batch_size):
            sel = idx[pos:pos + self.batch_size]
            bd = d.index_select(0, sel.to(d.device))
            bt = t.index_select(0, sel.to(t.device))
            if self.pin and not bd.is_cuda:
                bd, bt = bd.pin_memory(), bt.pin_memory()
            yield Tensor(_data=bd), Tensor(_data=bt)

    __iter__ = iter

    def __repr__(self):
        return "DataLoader(samples=%d, batch_size=%d, batches=%d)" % (
            self.n_samples, self.batch_size, self.num_batches())
