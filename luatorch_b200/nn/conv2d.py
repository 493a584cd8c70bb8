"""2-d convolution lowered to a GEMM (lua/luatorch/nn/conv2d.lua:17-120).

Same interface and layouts as the reference: weight [out_c, in_c*k*k] (randn*sqrt(2/fan_in)),
bias [out_c]; `forward(input, batch, height, width)` takes a flat NCHW input and returns
`(out, out_h, out_w)` with `out` shaped [batch*out_h*out_w, out_c] (NHWC-flat).

Beyond the reference: the gradient w.r.t. the convolution input exists (col2im of
dY @ W), everything runs on the GPU (im2col / col2im kernels + tensor-core GEMMs with the bias
and an optional ReLU in the epilogue), and `to_nchw` / `to_nhwc` re-layout helpers let
convolutions be chained (the reference's output layout does not match its own input layout).
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import _backend as B
from .. import autograd
from ..tensor import Tensor
from .linear import write_param_grad
from .module import Module, compute_view, param


def _pad8(n: int) -> int:
    return (n + 7) // 8 * 8


class Conv2d(Module):
    def __init__(self, in_channels: int, out_channels: int, kernel_size: int, stride: int = 1,
                 padding: int = 0):
        self.in_channels = in_channels
        self.out_channels = out_channels
        self.kernel_size = kernel_size
        self.stride = stride or 1
        self.padding = padding or 0
        fan_in = in_channels * kernel_size * kernel_size
        self.weight = param([out_channels, fan_in], "randn", math.sqrt(2.0 / fan_in))
        self.bias = param([out_channels])

    def output_size(self, height: int, width: int):
        k, s, p = self.kernel_size, self.stride, self.padding
        return (height + 2 * p - k) // s + 1, (width + 2 * p - k) // s + 1

    def forward(self, input: Tensor, batch: int, height: int, width: int, act: Optional[str] = None):
        C, k, s, p = self.in_channels, self.kernel_size, self.stride, self.padding
        oh, ow = self.output_size(height, width)
        x = input._t
        weight, bias = self.weight, self.bias
        patch = C * k * k
        if x.is_cuda and (x.dtype == torch.bfloat16 or weight._compute is not None):
            out = self._forward_tc(input, batch, height, width, oh, ow, act)
            return out, oh, ow
        cols = B.im2col(x, batch, C, height, width, k, s, p)                # [rows, patch]
        y = B.add_broadcast(B.matmul(cols, B.transpose(weight._t.to(cols.dtype))),
                            bias._t.to(cols.dtype))
        out = Tensor(_data=y)

        def grad_fn(g):
            gt = g._t
            if weight.requires_grad:
                autograd.acc_grad(weight, B.matmul(B.transpose(gt), cols).to(weight._t.dtype))
            if bias.requires_grad:
                autograd.acc_grad(bias, B.column_sum(gt).to(bias._t.dtype))
            if input.requires_grad:
                dcols = B.matmul(gt, weight._t.to(gt.dtype))
                dx = B.col2im(dcols, batch, C, height, width, k, s, p)
                autograd.acc_grad(input, dx.reshape(input._t.shape))

        autograd.record("conv2d", [input, weight, bias], out, grad_fn)
        if act == "relu":
            out = autograd.relu(out)
        return out, oh, ow

    def _forward_tc(self, input, batch, height, width, oh, ow, act):
        C, k, s, p = self.in_channels, self.kernel_size, self.stride, self.padding
        x = input._t
        if x.dtype != torch.bfloat16:
            x = B.cast(x, torch.bfloat16)
        patch = C * k * k
        ld = _pad8(patch)
        cols = B.ext().im2col(x.reshape(-1), batch, C, height, width, k, s, p, ld)  # [rows, ld]
        w = compute_view(self.weight, x)
        if ld != patch:  # TMA needs 16-byte row strides: stage a column-padded copy
            wp = torch.zeros((self.out_channels, ld), device=x.device, dtype=torch.bfloat16)
            wp[:, :patch].copy_(w)
            w = wp
        b = compute_view(self.bias, x)
        rows = cols.shape[0]
        pre = None
        if act == "relu" and autograd.enabled:
            pre = torch.empty((rows, self.out_channels), device=x.device, dtype=torch.bfloat16)
        # out[rows, out_c] = cols[rows, patch] @ W^T ; W is [out_c, patch] = K-major operand B
        y = torch.empty((rows, self.out_channels), device=x.device, dtype=torch.bfloat16)
        C_ = B.ext()
        C_.gemm(cols, w, y, rows, self.out_channels, patch, ld, w.stride(0), self.out_channels,
                False, False, 1, 1, 0, 0, 0, 0, 0, 0, 1.0, False, b, 3 if act == "relu" else 0,
                None, 0, pre, None, 0, 0)
        out = Tensor(_data=y)
        weight, bias = self.weight, self.bias
        oc = self.out_channels

        def grad_fn(g):
            gt = g._t if g._t.dtype == torch.bfloat16 else g._t.to(torch.bfloat16)
            if act == "relu":
                gt = C_.unary_backward(B._UN["relu"], pre, gt)
            if weight.requires_grad:
                # dW[out_c, patch] = dY^T[out_c, rows] @ cols[rows, patch]
                def dw(o, acc):
                    C_.gemm(gt, cols, o, oc, patch, rows, oc, ld, o.stride(0), True, True, 1, 1,
                            0, 0, 0, 0, 0, 0, 1.0, acc, None, 0, None, 0, None, None, 0, 0)
                write_param_grad(weight, dw)
            if bias.requires_grad:
                write_param_grad(bias, lambda o, acc: B.column_sum(gt, o, acc))
            if input.requires_grad:
                # dcols[rows, patch] = dY[rows, out_c] @ W[out_c, patch]
                dcols = torch.empty((rows, ld), device=x.device, dtype=torch.bfloat16)
                C_.gemm(gt, w, dcols, rows, patch, oc, oc, w.stride(0), ld, False, True, 1, 1,
                        0, 0, 0, 0, 0, 0, 1.0, False, None, 0, None, 0, None, None, 0, 0)
                dx = C_.col2im(dcols[:, :patch], batch, C, height, width, k, s, p)
                autograd.acc_grad(input, dx.reshape(input._t.shape).to(input._t.dtype))

        autograd.record("conv2d", [input, weight, bias], out, grad_fn)
        return out

    def parameters(self):
        return [self.weight, self.bias]

    def __repr__(self):
        return "Conv2d(%d, %d, kernel=%d, stride=%d, pad=%d)" % (
            self.in_channels, self.out_channels, self.kernel_size, self.stride, self.padding)


def _relayout(x: Tensor, batch: int, channels: int, hw: int, to_nchw: bool) -> Tensor:
    out = Tensor(_data=B.relayout(x._t, batch, channels, hw, to_nchw))

    def grad_fn(g):
        if x.requires_grad:
            autograd.acc_grad(x, B.relayout(g._t, batch, channels, hw, not to_nchw).reshape(x._t.shape))

    autograd.record("relayout", [x], out, grad_fn)
    return out


def to_nchw(x: Tensor, batch: int, channels: int, hw: int) -> Tensor:
    """[batch*hw, channels] (a Conv2d output) -> flat NCHW (a Conv2d input)."""
    return _relayout(x, batch, channels, hw, True)


def to_nhwc(x: Tensor, batch: int, channels: int, hw: int) -> Tensor:
    return _relayout(x, batch, channels, hw, False)
