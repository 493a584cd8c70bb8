"""SGD with momentum and optional Nesterov update (lua/luatorch/optim/sgd.lua:15-73):
v = mu*v + g;  p -= lr*v   (nesterov: p -= lr*(mu*v + g)).  Defaults lr 0.01, momentum 0.9.

With a parameter arena the whole model is one fused launch that also refreshes the bf16
shadow weights; the reference has no CUDA kernel for SGD at all."""
from __future__ import annotations

from typing import Sequence

import torch

from .. import _backend as B
from ..parallel.arena import arena_of, storage_units
from ..tensor import Tensor
from .adam import _unit_grad


class SGD:
    @classmethod
    def new(cls, *args, **kwargs):
        """`X.new(...)` is `X(...)`, the reference's constructor spelling."""
        return cls(*args, **kwargs)

    def __init__(self, params: Sequence[Tensor], lr: float = None, momentum: float = None,
                 nesterov: bool = False):
        self.params = list(params)
        self.lr = 0.01 if lr is None else lr
        self.momentum = 0.9 if momentum is None else momentum
        self.nesterov = bool(nesterov)
        self.grad_scale = 1.0
        self.units = storage_units(self.params)
        arenas = {id(a): a for a in (arena_of(p) for p in self.params) if a is not None}
        self.arena = None
        if len(arenas) == 1 and all(arena_of(p) is not None for p in self.params):
            self.arena = next(iter(arenas.values()))
        if self.arena is not None:
            a = self.arena
            self.v_flat = torch.zeros(a.state_numel(), device=a.device, dtype=torch.float32)
            if a.state_shards is None:
                self.velocity = [self.v_flat[o:o + u.numel()].view(u._t.shape)
                                 for u, o in zip(a.units, a.offsets)]
            else:
                self.velocity = None     # sharded over the ranks; see state_dict()
        else:
            self.velocity = [torch.zeros_like(u._t, dtype=torch.float32) for u in self.units]

    def step(self) -> None:
        if self.arena is not None and self.arena.state_shards is not None:
            raise RuntimeError("optimizer state is sharded over the ranks: step() runs inside "
                               "the fused collective (distributed.DDP.attach(optimizer))")
        if self.arena is not None and self.arena.master.is_cuda:
            a = self.arena
            B.sgd_flat(a.master, a.shadow, a.grad, self.v_flat if self.momentum else None,
                       self.lr, self.momentum, self.nesterov, self.grad_scale)
            return
        for i, u in enumerate(self.units):
            g = _unit_grad(u, self.params)
            if g is None:
                continue
            p = u._t
            if self.velocity[i].device != p.device:
                self.velocity[i] = self.velocity[i].to(p.device)
            v = self.velocity[i]
            if p.is_cuda and p.is_contiguous() and p.dtype == torch.float32:
                gg = g.contiguous()
                if gg.dtype not in (torch.float32, torch.bfloat16):
                    gg = gg.float()
                B.ext().sgd_flat(p.view(-1), None, gg.view(-1), v.view(-1) if self.momentum else None,
                                 self.lr, self.momentum, self.nesterov, self.grad_scale)
            else:
                gf = g.to(torch.float32).reshape(p.shape) * self.grad_scale
                if self.momentum:
                    v.mul_(self.momentum).add_(gf)
                    upd = gf + self.momentum * v if self.nesterov else v
                else:
                    upd = gf
                p.sub_((self.lr * upd).to(p.dtype))
            if u._compute is not None:
                u._compute.copy_(u._t)

    def reset(self) -> None:
        if self.arena is not None:
            self.v_flat.zero_()
            return
        for v in self.velocity:
            v.zero_()

    def set_lr(self, lr: float) -> None:
        self.lr = lr

    def state_dict(self) -> dict:
        """With sharded state a COLLECTIVE: every rank calls it and receives the full velocity."""
        a = self.arena
        if a is not None and a.state_shards is not None:
            full = a.state_shards.gather(self.v_flat, a.total)
            return {"lr": self.lr, "velocity": [full[o:o + u.numel()].view(u._grad_buf.shape).cpu()
                                                for u, o in zip(a.units, a.offsets)]}
        return {"lr": self.lr, "velocity": [v.detach().cpu().clone() for v in self.velocity]}

    def load_state_dict(self, state: dict) -> None:
        self.lr = float(state["lr"])
        a = self.arena
        if a is not None and a.state_shards is not None:
            full = torch.zeros(a.total, device=self.v_flat.device, dtype=torch.float32)
            for u, o, src in zip(a.units, a.offsets, state["velocity"]):
                full[o:o + u.numel()].copy_(src.reshape(-1))
            a.state_shards.take(full, out=self.v_flat)
            return
        for dst, src in zip(self.velocity, state["velocity"]):
            dst.copy_(src.reshape(dst.shape))

    def __repr__(self):
        return "SGD(lr=%g, momentum=%g, nesterov=%s, params=%d)" % (
            self.lr, self.momentum, str(self.nesterov).lower(), len(self.params))
