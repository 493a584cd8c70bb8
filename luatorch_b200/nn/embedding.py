"""Token embedding: weight [vocab, dim] initialised randn * 0.02; forward gathers rows for a
tensor of ids (stored as floats in the reference, any integer dtype accepted here), backward
scatter-adds into a dense gradient (lua/luatorch/nn/embedding.lua:14-82).

CUDA: one gather kernel forward; backward is the deterministic counting-sort scatter-add
(no atomics), written in place into the parameter's gradient buffer."""
from __future__ import annotations

import sys

import torch

from .. import _backend as B
from ..utils import debug as _debug
from .. import autograd
from ..tensor import Tensor
from .module import Module, param


def embedding_backward_into(weight_p: Tensor, dy: torch.Tensor, ids: torch.Tensor):
    vocab, dim = weight_p._t.shape
    if dy.is_cuda:
        def compute(out, acc):
            B.ext().embedding_backward(dy if dy.is_contiguous() else dy.contiguous(), ids, out, acc)
        from .linear import write_param_grad
        write_param_grad(weight_p, compute)
    else:
        g = torch.zeros((vocab, dim), dtype=torch.float32)
        g.index_add_(0, ids.reshape(-1).long(), dy.float().reshape(-1, dim))
        autograd.acc_grad(weight_p, g.to(weight_p._t.dtype))


class Embedding(Module):
    def __init__(self, vocab_size: int, embedding_dim: int):
        self.vocab_size = vocab_size
        self.embedding_dim = embedding_dim
        self.weight = param([vocab_size, embedding_dim], "randn", 0.02)

    def forward(self, input: Tensor) -> Tensor:
        ids = input._t.reshape(-1)
        w = self.weight
        if w._t.is_cuda:
            if not ids.is_cuda:
                ids = ids.cuda()
            table = w._compute if w._compute is not None else w._t
            y, err = B.ext().embedding_forward(table, B._labels(ids), None, 1)
            _debug.check_index_word(err, "Embedding: token id")
            out = Tensor(_data=y)
        else:
            idx = ids.long()
            if idx.numel() and (int(idx.min()) < 0 or int(idx.max()) >= self.vocab_size):
                print("luatorch error: embedding index out of range", file=sys.stderr)
                idx = idx.clamp(0, self.vocab_size - 1)
            out = Tensor(_data=w._t.index_select(0, idx))
            ids = idx

        def grad_fn(g):
            if w.requires_grad:
                embedding_backward_into(w, g._t, ids if not g._t.is_cuda else B._labels(ids))

        autograd.record("embedding", [w], out, grad_fn)
        return out

    def parameters(self):
        return [self.weight]

    def __repr__(self):
        return "Embedding(%d, %d)" % (self.vocab_size, self.embedding_dim)
