"""BatchNorm1d over [batch, features] (lua/luatorch/nn/batchnorm.lua:14-203): batch
statistics + running mean / var (momentum 0.1, biased variance) while training, running
statistics in eval; gamma ones, beta zeros.

Normalising every feature over the batch is a LayerNorm over the rows of the TRANSPOSED
input, so the layer is built from kernels that already exist: tiled transpose, the fused row
LayerNorm forward / backward (unit gamma, zero beta), a per-column affine and the
deterministic column sums.  The reference loops over elements in Lua.  Running statistics
are exposed through `buffers()` so checkpoints of the training state can include them (the
reference leaves them out of `parameters()` and therefore never saves them)."""
from __future__ import annotations

import torch

from .. import _backend as B
from .. import autograd
from ..tensor import Tensor
from .module import Module, param


class BatchNorm1d(Module):
    def __init__(self, num_features: int, eps: float = 1e-5, momentum: float = 0.1):
        self.num_features = num_features
        self.eps = eps or 1e-5
        self.momentum = momentum if momentum is not None else 0.1
        self.training = True
        self.gamma = param([num_features], "ones")
        self.beta = param([num_features])
        self.running_mean = Tensor([num_features])
        self.running_var = Tensor([num_features]).ones()

    def _moved(self):
        dev = self.gamma._t.device
        self.running_mean._t = self.running_mean._t.to(dev)
        self.running_var._t = self.running_var._t.to(dev)

    def buffers(self):
        return [self.running_mean, self.running_var]

    def forward(self, input: Tensor) -> Tensor:
        x = input._t
        n, f = x.shape
        dev, dt = x.device, x.dtype
        gamma, beta = self.gamma, self.beta
        g = gamma._t.to(dt)
        b = beta._t.to(dt)
        if self.training:
            xt = B.transpose(x)                                         # [features, batch]
            ones = torch.ones(n, device=dev, dtype=dt)
            zeros = torch.zeros(n, device=dev, dtype=dt)
            xhat_t, mean, rstd = B.layernorm(xt, ones, zeros, self.eps)  # stats per feature
            xhat = B.transpose(xhat_t)
            var = 1.0 / (rstd * rstd) - self.eps
            m = self.momentum
            self.running_mean._t.mul_(1.0 - m).add_(mean.to(self.running_mean._t.dtype), alpha=m)
            self.running_var._t.mul_(1.0 - m).add_(var.to(self.running_var._t.dtype), alpha=m)
        else:
            rstd = torch.rsqrt(self.running_var._t.float() + self.eps)
            mean = self.running_mean._t.float()
            xhat = B.affine_cols(x, rstd.to(dt), (-mean * rstd).to(dt))
            xt = None
        out = Tensor(_data=B.affine_cols(xhat, g, b))
        training = self.training

        def grad_fn(grad):
            dy = grad._t.to(dt)
            if gamma.requires_grad:
                autograd.acc_grad(gamma, B.column_sum(B.binary("mul", dy, xhat)).to(gamma._t.dtype))
            if beta.requires_grad:
                autograd.acc_grad(beta, B.column_sum(dy).to(beta._t.dtype))
            if input.requires_grad:
                dxhat = B.affine_cols(dy, g)
                if training:
                    dg = torch.empty(n, device=dev, dtype=torch.float32)
                    db = torch.empty(n, device=dev, dtype=torch.float32)
                    dxt = B.layernorm_backward(xt, B.transpose(dxhat), ones, mean, rstd, dg, db)
                    autograd.acc_grad(input, B.transpose(dxt))
                else:
                    autograd.acc_grad(input, B.affine_cols(dxhat, rstd.to(dt)))

        autograd.record("batchnorm1d", [input, gamma, beta], out, grad_fn)
        return out

    def parameters(self):
        return [self.gamma, self.beta]

    def num_params(self):
        return 2 * self.num_features

    def __repr__(self):
        return "BatchNorm1d(%d, eps=%g, momentum=%g)" % (self.num_features, self.eps, self.momentum)
