"""Mixed-precision helpers: `GradScaler` (lua/luatorch/cuda/amp.lua) and the bf16 compute
switch the reference lacks.

GradScaler keeps the reference's numbers (scale 65536, growth x2 every 2000 clean steps,
backoff x0.5) and call sequence `scale_loss -> backward -> step(optimizer) -> update()`.
Differences: `scale_loss` is a tracked op, so the scaled loss really drives the backward pass
(the reference multiplies outside the tape and its losses ignore the incoming gradient, so
scaling has no effect there); unscale + inf/nan detection is one fused kernel per gradient
writing a device-resident flag that the optimizer kernel consumes (`skip_flag`), so the only
host read per step is that flag in `update()`.

`autocast_bf16(model)` puts a model's parameters into a flat arena with an fp32 master copy
and a bf16 shadow that all kernels read: the "bf16 compute / fp32 master" mode.
"""
from __future__ import annotations

import torch

from .. import _backend as B
from .. import autograd
from ..parallel.arena import ParamArena
from ..tensor import Tensor


class GradScaler:
    def __init__(self, init_scale: float = None, growth_factor: float = None,
                 backoff_factor: float = None, growth_interval: int = None):
        self.scale = 65536.0 if init_scale is None else init_scale
        self.growth_factor = 2.0 if growth_factor is None else growth_factor
        self.backoff_factor = 0.5 if backoff_factor is None else backoff_factor
        self.growth_interval = 2000 if growth_interval is None else growth_interval
        self.growth_tracker = 0
        self.found_inf = False
        self._current_scale = self.scale
        self._flag = None

    @classmethod
    def new(cls, *a, **k):
        return cls(*a, **k)

    def scale_loss(self, loss: Tensor) -> Tensor:
        scale = self.scale
        self._current_scale = scale
        out = Tensor.mul_scalar(loss, scale)

        def grad_fn(g):
            if loss.requires_grad:
                autograd.acc_grad(loss, Tensor.mul_scalar(g, scale))

        autograd.record("scale_loss", [loss], out, grad_fn)
        return out

    def step(self, optimizer) -> None:
        inv = 1.0 / self._current_scale
        self.found_inf = False
        arena = getattr(optimizer, "arena", None)
        if arena is not None and arena.grad.is_cuda:
            if self._flag is None:
                self._flag = torch.zeros(1, device=arena.grad.device, dtype=torch.int32)
            self._flag.zero_()
            # one pass over the whole gradient arena: detect non-finite values; the unscale
            # itself is folded into the optimizer kernel's grad_scale
            B.ext().check_finite_scale(arena.grad, inv, False, self._flag)
            prev_scale, prev_flag = optimizer.grad_scale, optimizer.skip_flag
            optimizer.grad_scale = prev_scale * inv
            optimizer.skip_flag = self._flag
            try:
                optimizer.step()
            finally:
                optimizer.grad_scale, optimizer.skip_flag = prev_scale, prev_flag
            self._pending_flag = True
            return
        self._pending_flag = False
        for p in optimizer.params:
            if p.grad is None:
                continue
            g = p.grad._t
            if g.is_cuda and g.is_contiguous() and g.dtype in B._KERNEL_DTYPES:
                flag = torch.zeros(1, device=g.device, dtype=torch.int32)
                B.ext().check_finite_scale(g, inv, True, flag)
                if int(flag.item()):
                    self.found_inf = True
            else:
                g.mul_(inv)
                if not bool(torch.isfinite(g).all()):
                    self.found_inf = True
        if not self.found_inf:
            optimizer.step()

    def update(self) -> None:
        if getattr(self, "_pending_flag", False):
            self.found_inf = bool(int(self._flag.item()))
            self._pending_flag = False
        if self.found_inf:
            self.scale *= self.backoff_factor
            self.growth_tracker = 0
        else:
            self.growth_tracker += 1
            if self.growth_tracker >= self.growth_interval:
                self.scale *= self.growth_factor
                self.growth_tracker = 0

    def get_scale(self) -> float:
        return self.scale

    def state_dict(self):
        return {"scale": self.scale, "growth_tracker": self.growth_tracker}

    def load_state_dict(self, s):
        self.scale, self.growth_tracker = float(s["scale"]), int(s["growth_tracker"])

    def __repr__(self):
        return "GradScaler(scale=%.1f, growth=%d/%d)" % (self.scale, self.growth_tracker,
                                                         self.growth_interval)


def autocast_bf16(model, device: str = "cuda", grad_dtype: torch.dtype = torch.bfloat16,
                  allocator=None) -> ParamArena:
    """Move `model` to `device` in bf16-compute / fp32-master mode; returns the arena."""
    if device == "cuda":
        model.cuda()
    arena = ParamArena(model.parameters(), device=device, compute_dtype=torch.bfloat16,
                       grad_dtype=grad_dtype, allocator=allocator)
    return arena
