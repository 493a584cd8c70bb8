"""CUDA-graph replay of a whole training step.

A launch-bound step (a small MLP issues some thirty kernels of a few microseconds each) spends
most of its time in host launch overhead.  `GraphedStep` captures ONE step — zero the
gradients, forward, loss, backward, gradient synchronisation, optimizer update — into a CUDA
graph and replays it with a single launch:

    step = lf.cuda.GraphedStep(one_step, opt, inputs=(x, y))
    for xb, yb in loader:
        loss = step(xb, yb)          # copies xb, yb into x, y, replays, returns the loss Tensor

What changes from step to step cannot be a launch argument of a replayed graph, so those
scalars live in device memory and one single-thread kernel refreshes them before each replay:
the learning rate (schedulers keep working), Adam's bias corrections 1-beta^t, and the Philox
offset of the dropout masks (each replay draws fresh masks, and backward regenerates the
forward's).  Everything else a step needs — tile choices, split-K workspaces, the autograd
tape's closures — is fixed at capture time, so shapes must stay the same; build a second
GraphedStep for another batch shape.

Several ranks: the fused gradient collectives number themselves from a counter in their
signal pad and read lr / bias corrections from the same device words, so the captured step
(forward, backward, the per-bucket reduce + optimizer kernels on the side stream) replays on
every rank; all ranks must call the step the same number of times.

Limit: parameters in a flat arena (wrap the model in `distributed.DDP`, which at one rank is
just the arena plus the fused optimizer launch).  The reference has no counterpart; it issues
every op from LuaJIT (lua/luatorch/autograd.lua:52-93, lua/luatorch/optim/adam.lua:44-86).
"""
from __future__ import annotations

import os
from typing import Callable, Optional, Sequence

import torch

from .. import _backend as B
from ..tensor import Tensor


class GraphedStep:
    """Capture `step_fn()` once, replay it on every call.

    step_fn   -- runs one complete training step on static input tensors and returns the loss
                 Tensor (or any Tensor / tuple of Tensors to read back after a replay).
    optimizer -- the Adam / AdamW / SGD instance that step_fn steps; its `t` and `lr` are read
                 before every replay.
    inputs    -- the static input Tensors that step_fn reads; `__call__(*new)` copies new
                 batches into them.
    warmup    -- eager steps run before the capture (they are real training steps: kernels,
                 workspaces and allocator pools reach their steady state).
    pdl       -- keep programmatic dependent launch on inside the captured graph (default:
                 off, or LT_GRAPH_PDL=1 in the environment).
    """

    def __init__(self, step_fn: Callable[[], object], optimizer, inputs: Sequence[Tensor] = (),
                 warmup: int = 3, pdl: Optional[bool] = None):
        if pdl is None:
            pdl = os.environ.get("LT_GRAPH_PDL", "0") == "1"
        if not torch.cuda.is_available():
            raise RuntimeError("GraphedStep needs a CUDA device")
        if getattr(optimizer, "arena", None) is None:
            raise ValueError("GraphedStep needs the optimizer's parameters in a flat arena "
                             "(wrap the model in distributed.DDP before building the optimizer)")
        self.step_fn = step_fn
        self.optimizer = optimizer
        self.inputs = list(inputs)
        self.uses_optimizer = False     # set by the optimizer launch helpers during the capture
        dev = self.inputs[0]._t.device if self.inputs else torch.device("cuda")
        self.dyn_opt = torch.zeros(4, device=dev, dtype=torch.float32)
        self.dyn_off = torch.zeros(1, device=dev, dtype=torch.int64)
        self.replays = 0

        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(max(1, warmup)):
                step_fn()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()

        t_before = getattr(optimizer, "t", None)
        self._off0 = B.rng_state()["offset"]
        self._write_scalars(first=True)
        self.graph = torch.cuda.CUDAGraph()
        B._graph_capture = self
        if not pdl:
            B.ext().set_pdl(0)
        try:
            # with several ranks the process group's watchdog thread polls CUDA events while
            # this thread captures: thread-local mode keeps its calls out of the capture
            from .. import distributed as dist_mod
            mode = "thread_local" if dist_mod.world_size() > 1 else "global"
            with torch.cuda.graph(self.graph, capture_error_mode=mode):
                self.output = step_fn()
        finally:
            B._graph_capture = None
            if not pdl:
                B.ext().set_pdl(-1)
        self._span = B.rng_state()["offset"] - self._off0
        if t_before is not None:
            optimizer.t = t_before          # the capture ran the host code only, no kernels

    # ------------------------------------------------------------------ replay
    def _write_scalars(self, first: bool = False) -> None:
        opt = self.optimizer
        t = getattr(opt, "t", 0) + 1
        b1, b2 = getattr(opt, "beta1", 0.0), getattr(opt, "beta2", 0.0)
        if first:
            shift = 0
        else:
            st = B.rng_state()
            shift = st["offset"] - self._off0
            if self._span:
                B.next_philox(4 * self._span)     # reserve this replay's slice of the counter space
        B.ext().set_step_scalars(self.dyn_opt, opt.lr, 1.0 - b1 ** t, 1.0 - b2 ** t, self.dyn_off,
                                 shift)

    def __call__(self, *new_inputs):
        if new_inputs:
            if len(new_inputs) != len(self.inputs):
                raise ValueError("expected %d inputs" % len(self.inputs))
            for dst, src in zip(self.inputs, new_inputs):
                s = src._t if isinstance(src, Tensor) else src
                dst._t.copy_(s, non_blocking=True)
        self._write_scalars()
        self.graph.replay()
        if self.uses_optimizer and hasattr(self.optimizer, "t"):
            self.optimizer.t += 1           # the replay ran one optimizer update
        self.replays += 1
        return self.output

    def __repr__(self):
        return "GraphedStep(replays=%d, philox_span=%d)" % (self.replays, self._span)
