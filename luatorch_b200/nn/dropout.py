"""Dropout (lua/luatorch/nn/dropout.lua:15-59): zero each element with probability p
(default 0.5) while training, scale survivors by 1/(1-p); identity in eval.

CUDA: the mask is never stored; forward and backward regenerate it from the same Philox
(seed, offset) pair inside the kernel."""
from __future__ import annotations

from .. import _backend as B
from .. import autograd
from ..tensor import Tensor
from .module import Module


class Dropout(Module):
    def __init__(self, p: float = 0.5):
        self.p = 0.5 if p is None else p
        self.training = True

    def forward(self, input: Tensor) -> Tensor:
        if not self.training or self.p <= 0.0:
            return input
        p = self.p
        y, ctx = B.dropout(input._t, p)
        out = Tensor(_data=y)

        def grad_fn(g):
            if input.requires_grad:
                autograd.acc_grad(input, B.dropout_backward(g._t, p, ctx))

        autograd.record("dropout", [input], out, grad_fn)
        return out

    def __repr__(self):
        return "Dropout(p=%g)" % self.p
