"""Reading per-step device scalars (the loss) on the host without draining the GPU.

`loss.item()` right after a step blocks the host until that step has finished, so the next
step's input copy and launches start on an idle GPU.  `ScalarFetcher.push(loss)` enqueues an
asynchronous device-to-host copy into pinned memory instead and hands back the value pushed
`depth` calls earlier, whose copy has finished long before: every step's value still reaches
the host, one step late, while the next step is already queued behind the running one.  The
reference reads its loss synchronously for the logger (examples/gpt.lua:176-183,
lua/luatorch/utils/logger.lua:29-60)."""
from __future__ import annotations

from collections import deque
from typing import List, Optional

import torch

from ..tensor import Tensor


class ScalarFetcher:
    def __init__(self, depth: int = 1, device: Optional[torch.device] = None):
        if depth < 0:
            raise ValueError("depth must be >= 0")
        self.depth = depth
        self.cuda = torch.cuda.is_available() and (device is None or torch.device(device).type == "cuda")
        self._pending = deque()     # (slot index, event) oldest first
        self._free: List[int] = []
        self._slots = None
        if self.cuda:
            self._slots = torch.zeros(depth + 1, dtype=torch.float32).pin_memory()
            self._free = list(range(depth + 1))
        self._host = deque()        # CPU fallback: plain values

    def push(self, value) -> Optional[float]:
        """Queue `value` (a one-element Tensor) for reading; returns the value queued `depth`
        calls ago, or None while the pipeline fills."""
        t = value._t if isinstance(value, Tensor) else value
        if not (self.cuda and t.is_cuda):
            self._host.append(float(t.reshape(-1)[0].item()))
            return self._host.popleft() if len(self._host) > self.depth else None
        slot = self._free.pop()
        self._slots[slot:slot + 1].copy_(t.detach().reshape(-1)[:1].float(), non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._pending.append((slot, ev))
        if len(self._pending) > self.depth:
            return self._pop()
        return None

    def _pop(self) -> float:
        slot, ev = self._pending.popleft()
        ev.synchronize()
        v = float(self._slots[slot])
        self._free.append(slot)
        return v

    def drain(self) -> List[float]:
        """Wait for and return every value still in flight, oldest first."""
        out = list(self._host)
        self._host.clear()
        while self._pending:
            out.append(self._pop())
        return out
