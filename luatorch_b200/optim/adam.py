"""Adam and AdamW (lua/luatorch/optim/adam.lua, adamw.lua).

Same update rule and defaults: lr 1e-3, betas 0.9 / 0.999, eps 1e-8; AdamW applies the
decoupled decay p *= 1 - lr*wd BEFORE the Adam update, default weight_decay 0.01, and skips
it for the tensors listed in `no_decay_keys` (adamw.lua:19-49, 51-102).

Execution: when the parameters live in a flat arena the whole model is updated by ONE kernel
launch over (master fp32, shadow bf16, grad, m, v) with a per-segment decay table; otherwise
one fused launch per storage tensor on CUDA, plain tensor math on CPU.  The reference launches
once per parameter on CUDA and runs 11 tensor ops with 8 temporaries per parameter on CPU.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from .. import _backend as B
from ..parallel.arena import ParamArena, arena_of, storage_units
from ..tensor import Tensor


def _unit_grad(u: Tensor, params: Sequence[Tensor]) -> Optional[torch.Tensor]:
    """Gradient of a storage unit: its own, or the slices' gradients stitched together."""
    if u.grad is not None:
        return u.grad._t
    parts = [p for p in params if p._base is u]
    if not parts or all(p.grad is None for p in parts):
        return None
    g = torch.zeros(u._t.shape, device=u._t.device, dtype=u._t.dtype)
    for p in parts:
        if p.grad is not None:
            lo, hi = p._base_slice
            g[:, lo:hi] = p.grad._t.to(g.dtype)
    return g


class Adam:
    decoupled = False

    @classmethod
    def new(cls, *args, **kwargs):
        """`X.new(...)` is `X(...)`, the reference's constructor spelling."""
        return cls(*args, **kwargs)

    def __init__(self, params: Sequence[Tensor], lr: float = None, beta1: float = None,
                 beta2: float = None, epsilon: float = None):
        self.params = list(params)
        self.lr = 0.001 if lr is None else lr
        self.beta1 = 0.9 if beta1 is None else beta1
        self.beta2 = 0.999 if beta2 is None else beta2
        self.epsilon = 1e-8 if epsilon is None else epsilon
        self.weight_decay = 0.0
        self.no_decay = set()
        self.t = 0
        self.grad_scale = 1.0          # multiplied into gradients (1/world, 1/loss scale)
        self.skip_flag = None          # device int flag: nonzero => skip the step (overflow)
        self._setup_state()

    # ------------------------------------------------------------------ state
    def _setup_state(self):
        self.units = storage_units(self.params)
        arenas = {id(a): a for a in (arena_of(p) for p in self.params) if a is not None}
        self.arena: Optional[ParamArena] = None
        if len(arenas) == 1 and all(arena_of(p) is not None for p in self.params):
            self.arena = next(iter(arenas.values()))
        if self.arena is not None:
            a = self.arena
            # with memory-sharded state (distributed.DDP mode "sharded") the moments cover only
            # this rank's slices of the arena: 1/world of its length
            n_state = a.state_numel()
            self.m_flat = torch.zeros(n_state, device=a.device, dtype=torch.float32)
            self.v_flat = torch.zeros(n_state, device=a.device, dtype=torch.float32)
            if a.state_shards is None:
                self.m = [self.m_flat[o:o + u.numel()].view(u._t.shape) for u, o in zip(a.units, a.offsets)]
                self.v = [self.v_flat[o:o + u.numel()].view(u._t.shape) for u, o in zip(a.units, a.offsets)]
            else:
                self.m = self.v = None      # per-tensor views exist only after a gather
            self._segments = None
        else:
            self.m = [torch.zeros_like(u._t, dtype=torch.float32) for u in self.units]
            self.v = [torch.zeros_like(u._t, dtype=torch.float32) for u in self.units]

    def _decay_of(self, u: Tensor) -> float:
        if not self.decoupled or self.weight_decay == 0.0:
            return 0.0
        if id(u) in self.no_decay:
            return 0.0
        parts = [p for p in self.params if p._base is u]
        if parts and all(id(p) in self.no_decay for p in parts):
            return 0.0
        return self.weight_decay

    def segments(self):
        if self._segments is None:
            self._segments = self.arena.segments(self._decay_of)
        return self._segments

    # ------------------------------------------------------------------ step
    def step(self) -> None:
        self.t += 1
        bc1 = 1.0 - self.beta1 ** self.t
        bc2 = 1.0 - self.beta2 ** self.t
        if self.arena is not None:
            a = self.arena
            if a.state_shards is not None:
                raise RuntimeError("optimizer state is sharded over the ranks: step() runs inside "
                                   "the fused collective (distributed.DDP.attach(optimizer))")
            seg_end, seg_wd = self.segments()
            if a.master.is_cuda:
                B.adamw_flat(a.master, a.shadow, a.grad, self.m_flat, self.v_flat, seg_end,
                             seg_wd, self.lr, self.beta1, self.beta2, self.epsilon, bc1, bc2,
                             self.grad_scale, self.skip_flag)
                return
        for i, u in enumerate(self.units):
            g = _unit_grad(u, self.params)
            if g is None:
                continue
            wd = self._decay_of(u)
            p, m, v = u._t, self.m[i], self.v[i]
            if p.is_cuda and p.is_contiguous() and p.dtype == torch.float32:
                if self.skip_flag is not None and int(self.skip_flag.item()):
                    continue
                if not m.is_cuda:
                    self.m[i], self.v[i] = m.cuda(), v.cuda()
                    m, v = self.m[i], self.v[i]
                gg = g if self.grad_scale == 1.0 else B.scalar_op("mul", g, self.grad_scale)
                if gg.dtype not in (torch.float32, torch.bfloat16):
                    gg = gg.float()
                B.adam_step(p, gg.contiguous(), m, v, self.lr, self.beta1, self.beta2,
                            self.epsilon, bc1, bc2, wd)
            else:
                if m.device != p.device:
                    self.m[i], self.v[i] = m.to(p.device), v.to(p.device)
                    m, v = self.m[i], self.v[i]
                gg = g.to(torch.float32) * self.grad_scale if self.grad_scale != 1.0 else g.to(torch.float32)
                pf = p if p.dtype == torch.float32 else p.float()
                B.adam_step(pf, gg.reshape(pf.shape), m, v, self.lr, self.beta1, self.beta2,
                            self.epsilon, bc1, bc2, wd)
                if pf is not p:
                    p.copy_(pf)
            if u._compute is not None:
                u._compute.copy_(u._t)

    def reset(self) -> None:
        self.t = 0
        if self.arena is not None:
            self.m_flat.zero_()
            self.v_flat.zero_()
            return
        for m, v in zip(self.m, self.v):
            m.zero_()
            v.zero_()

    def set_lr(self, lr: float) -> None:
        self.lr = lr

    # ------------------------------------------------------------------ (de)serialisation
    def state_dict(self) -> dict:
        """Moments per storage tensor, on the CPU.  With sharded state this is a COLLECTIVE:
        every rank calls it and every rank receives the full moments."""
        a = self.arena
        if a is not None and a.state_shards is not None:
            out = {"t": self.t, "lr": self.lr}
            for key, flat in (("m", self.m_flat), ("v", self.v_flat)):
                full = a.state_shards.gather(flat, a.total)
                out[key] = [full[o:o + u.numel()].view(u._grad_buf.shape).cpu()
                            for u, o in zip(a.units, a.offsets)]
                del full
            return out
        return {"t": self.t, "lr": self.lr, "m": [m.detach().cpu().clone() for m in self.m],
                "v": [v.detach().cpu().clone() for v in self.v]}

    def load_state_dict(self, state: dict) -> None:
        self.t = int(state["t"])
        self.lr = float(state["lr"])
        a = self.arena
        if a is not None and a.state_shards is not None:
            # every rank holds the full saved moments and keeps its own slices
            for key, flat in (("m", self.m_flat), ("v", self.v_flat)):
                full = torch.zeros(a.total, device=flat.device, dtype=torch.float32)
                for u, o, src in zip(a.units, a.offsets, state[key]):
                    full[o:o + u.numel()].copy_(src.reshape(-1))
                a.state_shards.take(full, out=flat)
                del full
            return
        for dst, src in zip(self.m, state["m"]):
            dst.copy_(src.reshape(dst.shape))
        for dst, src in zip(self.v, state["v"]):
            dst.copy_(src.reshape(dst.shape))

    def __repr__(self):
        return "Adam(lr=%g, beta1=%g, beta2=%g, eps=%g, params=%d)" % (
            self.lr, self.beta1, self.beta2, self.epsilon, len(self.params))


class AdamW(Adam):
    decoupled = True

    def __init__(self, params: Sequence[Tensor], lr: float = None, beta1: float = None,
                 beta2: float = None, epsilon: float = None, weight_decay: float = None,
                 no_decay_keys: Optional[Sequence[Tensor]] = None):
        super().__init__(params, lr, beta1, beta2, epsilon)
        self.weight_decay = 0.01 if weight_decay is None else weight_decay
        self.no_decay = {id(p) for p in (no_decay_keys or [])}

    def __repr__(self):
        return "AdamW(lr=%g, beta1=%g, beta2=%g, eps=%g, wd=%g, params=%d)" % (
            self.lr, self.beta1, self.beta2, self.epsilon, self.weight_decay, len(self.params))
