"""Activation layers ReLU / Sigmoid / Tanh / GELU / SiLU (lua/luatorch/nn/activation.lua).

Forward and backward are one vectorised kernel each on CUDA; the reference computes the GELU
backward per element in Lua on the CPU (activation.lua:100-126)."""
from __future__ import annotations

from .. import _backend as B
from .. import autograd
from ..tensor import Tensor
from .module import Module


class _Activation(Module):
    op = ""

    def forward(self, input: Tensor) -> Tensor:
        out = Tensor(_data=B.unary(self.op, input._t))
        op = self.op

        def grad_fn(g):
            if input.requires_grad:
                autograd.acc_grad(input, B.unary_backward(op, input._t, g._t))

        autograd.record(op, [input], out, grad_fn)
        return out


class ReLU(_Activation):
    op = "relu"


class Sigmoid(_Activation):
    op = "sigmoid"


class Tanh(_Activation):
    op = "tanh"


class GELU(_Activation):
    op = "gelu"


class SiLU(_Activation):
    op = "silu"
