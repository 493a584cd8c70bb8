"""Shared pieces of the training entry points: device-timed step loop and rank-0 printing."""
from __future__ import annotations

import time

import torch

from .. import distributed as dist_mod


def is_rank0() -> bool:
    return dist_mod.rank() == 0


def log(*a):
    if is_rank0():
        print(*a, flush=True)


class StepTimer:
    """Device time of a window of steps (CUDA events), wall clock on CPU."""

    def __init__(self):
        self.cuda = torch.cuda.is_available()
        self.reset()

    def reset(self):
        if self.cuda:
            self.e0 = torch.cuda.Event(enable_timing=True)
            self.e0.record()
        self.t0 = time.perf_counter()

    def elapsed_ms(self) -> float:
        if self.cuda:
            e1 = torch.cuda.Event(enable_timing=True)
            e1.record()
            e1.synchronize()
            return self.e0.elapsed_time(e1)
        return (time.perf_counter() - self.t0) * 1e3


def max_over_ranks(ms: float) -> float:
    """A window's device time as the slowest rank saw it (one small all-reduce)."""
    if dist_mod.world_size() <= 1:
        return ms
    import torch.distributed as dist
    t = torch.tensor([ms], device="cuda" if torch.cuda.is_available() else "cpu", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
