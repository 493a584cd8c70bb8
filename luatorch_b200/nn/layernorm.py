"""LayerNorm over the last dimension: gamma ones, beta zeros, eps 1e-5, biased variance
(lua/luatorch/nn/layernorm.lua:15-126).  Forward and backward are the fused row kernels; the
reference module walks elements in Lua and never calls its own fused kernel."""
from __future__ import annotations


import torch

from .. import _backend as B
from .. import autograd
from ..tensor import Tensor
from .module import Module, compute_view, param


def layernorm_backward_into(x, dy, gamma_view, mean, rstd, gamma_p, beta_p, dx_add=None):
    """dx plus in-place (or accumulated) parameter gradients; shared with the fused
    transformer block."""
    gbuf, gacc = autograd.grad_target(gamma_p)
    bbuf, bacc = autograd.grad_target(beta_p)
    if gbuf is not None and bbuf is not None and gacc == bacc:
        dx = B.layernorm_backward(x, dy, gamma_view, mean, rstd, gbuf, bbuf, gacc, dx_add)
        autograd.grad_written(gamma_p)
        autograd.grad_written(beta_p)
        return dx
    cols = x.shape[-1]
    dg = torch.empty(cols, device=x.device, dtype=torch.float32)
    db = torch.empty(cols, device=x.device, dtype=torch.float32)
    dx = B.layernorm_backward(x, dy, gamma_view, mean, rstd, dg, db, False, dx_add)
    if gamma_p.requires_grad:
        autograd.acc_grad(gamma_p, dg.to(gamma_p._t.dtype))
    if beta_p.requires_grad:
        autograd.acc_grad(beta_p, db.to(beta_p._t.dtype))
    return dx


class LayerNorm(Module):
    def __init__(self, normalized_shape: int, eps: float = 1e-5):
        self.normalized_shape = normalized_shape
        self.eps = eps or 1e-5
        self.gamma = param([normalized_shape], "ones")
        self.beta = param([normalized_shape])

    def forward(self, input: Tensor) -> Tensor:
        x = input._t
        if x.is_cuda and self.gamma._compute is not None and x.dtype != torch.bfloat16:
            x = B.cast(x, torch.bfloat16)
        g = compute_view(self.gamma, x)
        b = compute_view(self.beta, x)
        y, mean, rstd = B.layernorm(x, g, b, self.eps)
        out = Tensor(_data=y)
        gamma, beta = self.gamma, self.beta

        def grad_fn(grad):
            dy = grad._t if grad._t.dtype == x.dtype else grad._t.to(x.dtype)
            # A residual branch may already have deposited its gradient on the input; the
            # kernel adds it while writing dx, which saves a separate elementwise pass.
            prior = None
            if (input.requires_grad and input.grad is not None and input._grad_buf is None
                    and input.grad._t.dtype == x.dtype and input.grad._t.shape == x.shape):
                prior = input.grad._t
            dx = layernorm_backward_into(x, dy, g, mean, rstd, gamma, beta, dx_add=prior)
            if input.requires_grad:
                if prior is not None:
                    input.grad = Tensor(_data=dx)
                else:
                    autograd.acc_grad(input, dx)

        autograd.record("layernorm", [input, gamma, beta], out, grad_fn)
        return out

    def parameters(self):
        return [self.gamma, self.beta]

    def __repr__(self):
        return "LayerNorm(%d, eps=%g)" % (self.normalized_shape, self.eps)
