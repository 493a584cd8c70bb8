"""Positional encodings (lua/luatorch/nn/positional.lua): SinusoidalPE (fixed table, gradient
passes through) and LearnedPE (weight [max_seq, dim], randn * 0.02, scatter-add backward).
`forward(input, seq_len)` adds row `t % seq_len` of the table to token `t` of a flattened
[batch*seq_len, dim] input.

On CUDA the add is the bias-broadcast kernel over the [batch, seq_len*dim] view and the
LearnedPE gradient is a deterministic column reduction over the batch."""
from __future__ import annotations

import math

import torch

from .. import _backend as B
from .. import autograd
from ..tensor import Tensor
from .module import Module, compute_view, param


def _add_positions(x: torch.Tensor, table: torch.Tensor, seq_len: int) -> torch.Tensor:
    dim = x.shape[-1]
    n_tokens = x.numel() // dim
    batch = n_tokens // seq_len
    rows = table[:seq_len].reshape(-1)
    if rows.dtype != x.dtype:
        rows = rows.to(x.dtype)
    return B.add_broadcast(x.reshape(batch, seq_len * dim), rows).reshape(x.shape)


class SinusoidalPE(Module):
    def __init__(self, max_seq_len: int, embed_dim: int):
        self.max_seq_len = max_seq_len
        self.embed_dim = embed_dim
        pos = torch.arange(max_seq_len, dtype=torch.float64).unsqueeze(1)
        i = torch.arange(embed_dim, dtype=torch.float64)
        div = torch.exp(-(i - (i % 2)) * math.log(10000.0) / embed_dim)
        angle = pos * div
        pe = torch.where((i % 2 == 0).unsqueeze(0), torch.sin(angle), torch.cos(angle))
        self.pe = Tensor(_data=pe.float())
        self._pe_cache = {}

    def _table(self, like: torch.Tensor) -> torch.Tensor:
        key = (like.device, like.dtype)
        t = self._pe_cache.get(key)
        if t is None:
            t = self.pe._t.to(device=like.device, dtype=like.dtype)
            self._pe_cache[key] = t
        return t

    def forward(self, input: Tensor, seq_len: int = None) -> Tensor:
        n_tokens = input.numel() // self.embed_dim
        seq_len = seq_len or n_tokens
        out = Tensor(_data=_add_positions(input._t, self._table(input._t), seq_len))

        def grad_fn(g):
            if input.requires_grad:
                autograd.acc_grad(input, g)

        autograd.record("positional", [input], out, grad_fn)
        return out

    def num_params(self):
        return 0

    def __repr__(self):
        return "SinusoidalPE(max_len=%d, dim=%d)" % (self.max_seq_len, self.embed_dim)


class LearnedPE(Module):
    def __init__(self, max_seq_len: int, embed_dim: int):
        self.max_seq_len = max_seq_len
        self.embed_dim = embed_dim
        self.weight = param([max_seq_len, embed_dim], "randn", 0.02)

    def forward(self, input: Tensor, seq_len: int = None) -> Tensor:
        dim = self.embed_dim
        n_tokens = input.numel() // dim
        seq_len = seq_len or n_tokens
        batch = n_tokens // seq_len
        w = self.weight
        out = Tensor(_data=_add_positions(input._t, compute_view(w, input._t), seq_len))

        def grad_fn(g):
            if input.requires_grad:
                autograd.acc_grad(input, g)
            if w.requires_grad:
                positional_backward_into(w, g._t, batch, seq_len)

        autograd.record("learned_pe", [input, w], out, grad_fn)
        return out

    def parameters(self):
        return [self.weight]

    def num_params(self):
        return self.max_seq_len * self.embed_dim

    def __repr__(self):
        return "LearnedPE(max_len=%d, dim=%d)" % (self.max_seq_len, self.embed_dim)


def positional_backward_into(w: Tensor, dy: torch.Tensor, batch: int, seq_len: int) -> None:
    dim = w._t.shape[1]
    if dy.is_cuda:
        from .linear import write_param_grad
        dyc = dy if dy.is_contiguous() else dy.contiguous()
        write_param_grad(w, lambda o, acc: B.ext().positional_backward(dyc, o, batch, seq_len, acc))
    else:
        g = torch.zeros(w._t.shape, dtype=torch.float32)
        g[:seq_len] = dy.float().reshape(batch, seq_len, dim).sum(0)
        autograd.acc_grad(w, g.to(w._t.dtype))
