"""NVTX ranges around the fused paths (forward, backward, each gradient bucket's reduce +
optimizer kernel, the optimizer join), for timeline tools that read NVTX.

Off by default: `enable()` or LT_NVTX=1 in the environment turns the ranges on; when off,
`range()` costs one flag test.  The reference has no profiler hooks at all (its timing is
os.clock() around a loop, tools/benchmark.lua:14-27)."""
from __future__ import annotations

import contextlib
import os

_on = os.environ.get("LT_NVTX", "0") == "1"
_impl = None
pushed = 0          # ranges opened so far (tests read this)


def _nvtx():
    global _impl
    if _impl is None:
        try:
            import torch.cuda.nvtx as n
            _impl = n
        except Exception:       # pragma: no cover - no CUDA build
            _impl = False
    return _impl


def enable(flag: bool = True) -> None:
    global _on
    _on = bool(flag)


def enabled() -> bool:
    return _on


def push(name: str) -> None:
    global pushed
    if _on:
        pushed += 1
        n = _nvtx()
        if n:
            try:
                n.range_push(name)
            except Exception:
                pass


def pop() -> None:
    if _on:
        n = _nvtx()
        if n:
            try:
                n.range_pop()
            except Exception:
                pass


@contextlib.contextmanager
def range(name: str):
    if not _on:
        yield
        return
    push(name)
    try:
        yield
    finally:
        pop()
