"""LayerNorm over the last dimension: gamma ones, beta zeros, eps 1e-5, biased variance
(lua/luatorch/nn/layernorm.lua:15-126).  Forward and backward are the fused row kernels; the
reference module walks elements in Lua and never calls its own fused kernel."""
from __future__ import annotations


import torch

from .. import _backend as B
from .. import autograd
from ..tensor import Tensor
from .module import Module, compute_view, param


def layernorm_backward_into(x, dy, gamma_view, mean, rstd, gamma_p, beta_p, dx_add=None,
                            bias_src=None):
    """dx plus in-place (or accumulated) parameter gradients; shared with the fused
    transformer block.  `bias_src` = [bias parameter, done flag] of the Linear whose output
    (plus residual) was normalised: dx is then the complete gradient of that output, and the
    kernels that write dx also sum its columns into the bias gradient."""
    gbuf, gacc = autograd.grad_target(gamma_p)
    bbuf, bacc = autograd.grad_target(beta_p)
    if (bias_src is not None and x.is_cuda and gbuf is not None and bbuf is not None
            and gacc == bacc):
        bias_p, flag = bias_src
        sbuf, sacc = autograd.grad_target(bias_p)
        if sbuf is not None and sbuf.dtype == gbuf.dtype and sbuf.is_contiguous() and not flag[0]:
            dx, done = B.ext().layernorm_backward_dxsum(
                B._k(x), B._k(dy), B._k(gamma_view), mean, rstd,
                None if dx_add is None else B._k(dx_add), gbuf, bbuf, gacc, sbuf, sacc)
            autograd.grad_written(gamma_p)
            autograd.grad_written(beta_p)
            if done:
                autograd.grad_written(bias_p)
                flag[0] = True
            return dx
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
        # The bias gradient of the Linear that produced `input` may ride on this backward only
        # if this LayerNorm is the FIRST consumer of `input` (its backward then runs after
        # every other consumer's, when input's gradient is complete): true exactly when the
        # node that produced `input` is still the last one on the tape.
        bias_src = None
        if (input._bias_src is not None and autograd.graph and input._node is not None
                and autograd.graph[-1] is input._node):
            bias_src = input._bias_src

        def grad_fn(grad):
            dy = grad._t if grad._t.dtype == x.dtype else grad._t.to(x.dtype)
            # A residual branch may already have deposited its gradient on the input; the
            # kernel adds it while writing dx, which saves a separate elementwise pass.
            prior = None
            if (input.requires_grad and input.grad is not None and input._grad_buf is None
                    and input.grad._t.dtype == x.dtype and input.grad._t.shape == x.shape):
                prior = input.grad._t
            # dx is the whole gradient of `input` when nothing else contributed, or when the
            # other contribution is added inside the kernel
            whole = input.requires_grad and (prior is not None or input.grad is None)
            dx = layernorm_backward_into(x, dy, g, mean, rstd, gamma, beta, dx_add=prior,
                                         bias_src=bias_src if whole else None)
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
