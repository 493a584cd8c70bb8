"""Module protocol shared by every layer: forward / __call__ / parameters / zero_grad /
num_params / train / eval / printable form, plus `X.new(...)` as an alias of `X(...)` so
both constructor spellings of the reference work (lua/luatorch/nn/init.lua:7-13)."""
from __future__ import annotations

from typing import List

import torch

from .. import autograd
from ..tensor import Tensor


class Module:
    training = True

    @classmethod
    def new(cls, *args, **kwargs):
        return cls(*args, **kwargs)

    def forward(self, *args, **kwargs):
        raise NotImplementedError

    def __call__(self, *args, **kwargs):
        return self.forward(*args, **kwargs)

    def parameters(self) -> List[Tensor]:
        return []

    def children(self) -> List["Module"]:
        return []

    def zero_grad(self) -> None:
        autograd.zero_grad(self.parameters())

    def num_params(self) -> int:
        return sum(p.numel() for p in self.parameters())

    def train(self):
        self.training = True
        for c in self.children():
            c.train()
        return self

    def eval(self):
        self.training = False
        for c in self.children():
            c.eval()
        return self

    def cuda(self):
        """Move every parameter to the GPU (in place, like Tensor.cuda)."""
        for p in self.parameters():
            p.cuda()
        for c in self.children():
            c._moved()
        self._moved()
        return self

    def cpu(self):
        for p in self.parameters():
            p.cpu()
        for c in self.children():
            c._moved()
        self._moved()
        return self

    def _moved(self) -> None:
        """Hook for modules holding non-parameter buffers."""

    def __repr__(self) -> str:
        return self.__class__.__name__ + "()"

    def __str__(self) -> str:
        return self.__repr__()


def param(shape, init: str = "zeros", scale: float = 1.0) -> Tensor:
    """Create a watched fp32 parameter."""
    t = Tensor(list(shape))
    if init == "randn":
        t.randn()
        if scale != 1.0:
            t._t.mul_(scale)
    elif init == "ones":
        t.ones()
    autograd.watch(t)
    return t


def compute_view(p: Tensor, like: torch.Tensor) -> torch.Tensor:
    """The storage of parameter `p` a kernel should read for activations shaped like `like`:
    the bf16 shadow when one exists and activations are bf16, else the parameter itself
    (cast on the fly if the dtypes differ)."""
    if p._compute is not None and like.dtype == p._compute.dtype:
        return p._compute
    if p._t.dtype == like.dtype:
        return p._t
    return p._t.to(like.dtype)
