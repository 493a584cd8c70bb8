"""Fully connected layer: out = input @ weight + bias.

Same parameter layout as the reference (lua/luatorch/nn/linear.lua:26-38, 82-88): weight is
[in_features, out_features] initialised randn * sqrt(2 / in), bias zeros [out]; parameter
order {weight, bias}.  That layout is what checkpoints store.

On CUDA with bf16 activations the whole layer is ONE tensor-core GEMM whose epilogue adds the
bias, optionally applies GELU / ReLU and adds a residual; backward is two GEMMs that read the
same buffers through transposed operand descriptors (no transposed copies) and write the
weight gradient straight into the parameter's gradient buffer.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import _backend as B
from .. import autograd
from ..tensor import Tensor
from .module import Module, compute_view, param

_ACT = {None: 0, "gelu": 1, "relu": 3}
_DACT = {"gelu": 2, "relu": 4}


def write_param_grad(p: Tensor, compute):
    """Run `compute(out, accumulate)` so that it writes the gradient of `p` into its
    preallocated buffer when there is one, else accumulate a fresh tensor."""
    buf, acc = autograd.grad_target(p)
    if buf is not None:
        compute(buf, acc)
        autograd.grad_written(p)
    else:
        g = torch.zeros(p._t.shape, device=p._t.device, dtype=p._t.dtype)
        compute(g, False)
        autograd.acc_grad(p, g)


class Linear(Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = True,
                 pad_out: bool = False):
        self.in_features = in_features
        self.out_features = out_features
        self.use_bias = bias is not False
        self.weight_storage = None
        if pad_out and out_features % 8 != 0:
            # Rows padded to a multiple of 8 columns (16 bytes of bf16) so TMA can address the
            # matrix; the parameter proper is the [in, out] view that checkpoints see.
            ld = (out_features + 7) // 8 * 8
            base = Tensor([in_features, ld])
            base._t[:, :out_features].copy_(
                Tensor([in_features, out_features]).randn()._t * math.sqrt(2.0 / in_features))
            autograd.watch(base)
            w = Tensor(_data=base._t[:, :out_features])
            w.requires_grad = True
            w._node = autograd.Node(w, "leaf", [])
            w._base, w._base_slice = base, (0, out_features)
            self.weight_storage, self.weight = base, w
        else:
            self.weight = param([in_features, out_features], "randn", math.sqrt(2.0 / in_features))
        self.bias = param([out_features]) if self.use_bias else None

    def _moved(self):
        if self.weight_storage is not None:
            base = self.weight_storage
            dev = self.weight._t.device
            if base._t.device != dev:
                base._t = base._t.to(dev)
            self.weight._t = base._t[:, :self.out_features]

    # ------------------------------------------------------------------ forward
    def forward(self, input: Tensor, residual: Optional[Tensor] = None,
                act: Optional[str] = None, sole_consumer: bool = False) -> Tensor:
        """`sole_consumer=True` promises that nothing else reads `input`; if `input` came out
        of a Linear with a fused activation, the activation's derivative is then applied in
        the epilogue of this layer's input-gradient GEMM instead of a separate pass."""
        x = input._t
        if x.is_cuda and (x.dtype == torch.bfloat16 or self.weight._compute is not None):
            return self._forward_tc(input, residual, act, sole_consumer)
        out = autograd.matmul(input, self.weight)
        if self.use_bias:
            mm = out
            out = Tensor.add_broadcast(mm, self.bias)
            bias = self.bias

            def grad_fn(g):
                if mm.requires_grad:
                    autograd.acc_grad(mm, g)
                if bias.requires_grad:
                    autograd.acc_grad(bias, B.column_sum(g._t))

            autograd.record("add_broadcast", [mm, bias], out, grad_fn)
        if act is not None:
            from . import activation
            out = {"gelu": activation.GELU, "relu": activation.ReLU}[act]()(out)
        if residual is not None:
            out = autograd.add(out, residual)
        return out

    def _forward_tc(self, input, residual, act, sole_consumer=False):
        x = input._t
        if x.dtype != torch.bfloat16:
            x = B.cast(x, torch.bfloat16)
        if x.stride(-1) != 1:
            x = x.contiguous()
        N = self.out_features
        storage = self.weight_storage
        w = compute_view(storage if storage is not None else self.weight, x)
        b = compute_view(self.bias, x) if self.use_bias else None
        M = x.shape[0]
        ldy = w.shape[1]                      # padded width when the weight rows are padded
        y = torch.empty((M, ldy), device=x.device, dtype=torch.bfloat16)[:, :N]
        pre = None
        if act is not None and autograd.enabled:
            pre = torch.empty((M, ldy), device=x.device, dtype=torch.bfloat16)[:, :N]
        B.gemm(x, w, bias=b, act=_ACT[act], aux_out=pre, out=y, n_valid=N,
               residual=None if residual is None else residual._t)
        out = Tensor(_data=y)
        if pre is not None:
            out._act_ctx = [act, pre, False]
        # out = x W + b + residual: the bias gradient is the column sum of out's gradient.  A
        # LayerNorm that consumes `out` first produces that very gradient in its backward
        # kernel and can sum its columns on the way (nn/layernorm.py); it then sets the flag.
        bias_folded = [False]
        if (residual is not None and act is None and self.use_bias and autograd.enabled
                and self.bias.requires_grad):
            out._bias_src = [self.bias, bias_folded]
        fuse_dact = (sole_consumer and input._act_ctx is not None and storage is None
                     and input._act_ctx[1].is_contiguous())
        weight, bias_p = (storage if storage is not None else self.weight), self.bias
        view_param = self.weight if storage is not None else None

        def grad_fn(g):
            gt = g._t if g._t.dtype == torch.bfloat16 else g._t.to(torch.bfloat16)
            if residual is not None and residual.requires_grad:
                autograd.acc_grad(residual, gt)
            if act is not None and not out._act_ctx[2]:
                gt = B.ext().unary_backward(B._UN[act], pre, gt)
            if gt.stride(-1) != 1:
                gt = gt.contiguous()
            dgrad_last = False      # the input-gradient GEMM is the kernel launched last
            if input.requires_grad:
                dgrad_last = input.grad is None
                if fuse_dact and input.grad is None:
                    in_act, in_pre, _ = input._act_ctx
                    autograd.acc_grad(input, B.gemm(gt, w, b_t=True, k_valid=N,
                                                    act=_DACT[in_act], aux_in=in_pre))
                    input._act_ctx[2] = True     # derivative already applied
                else:
                    autograd.acc_grad(input, B.gemm(gt, w, b_t=True, k_valid=N))
            if weight.requires_grad:
                if view_param is not None and view_param.grad is None:
                    weight.grad = None
                # dW reads x and g only and writes its own arena slot: independent of the
                # input-gradient GEMM just launched, so it may run in that kernel's tail
                write_param_grad(weight, lambda o, acc: B.gemm(x, gt, a_t=True, out=o,
                                                               accumulate=acc, n_valid=N,
                                                               overlap_prev=1 if dgrad_last else 0))
                if view_param is not None:
                    view_param.grad = Tensor(_data=weight.grad._t[:, :N])
            if bias_p is not None and bias_p.requires_grad and not bias_folded[0]:
                write_param_grad(bias_p, lambda o, acc: B.column_sum(gt, o, acc))

        autograd.record("linear", [input, weight, bias_p, residual, view_param], out, grad_fn)
        return out

    def parameters(self):
        return [self.weight, self.bias] if self.use_bias else [self.weight]

    def __repr__(self):
        return "Linear(%d -> %d%s)" % (self.in_features, self.out_features,
                                       "" if self.use_bias else ", bias=false")
