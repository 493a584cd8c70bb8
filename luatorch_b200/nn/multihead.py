"""Multi-head attention layers.

`MultiHeadAttention(embed_dim, num_heads)`: unmasked attention (lua/luatorch/nn/multihead.lua).
`FlashMultiHeadAttention(embed_dim, num_heads, causal)`: same projections with the flash
kernel and an optional causal mask (lua/luatorch/nn/flash_attention.lua).
Both: q/k/v projections without bias, output projection with bias, parameter order
{q.weight, k.weight, v.weight, out.weight, out.bias} (flash_attention.lua:150-158).

`forward(query, key=None, value=None, seq_len=None)` takes flattened [batch*seq_len, embed]
inputs; `seq_len` separates the sequences of a batch (default: one sequence).

What the reference gets wrong and this implementation does as intended: sequences of a batch
attend only to themselves, the causal mask is applied, and gradients flow through the
attention to q/k/v (the reference slices through fresh tensors and through a CPU round trip,
which cuts the tape; multihead.lua:80-138, flash_attention.lua:52-143).

Storage: the three projection weights are column slices of ONE fused [embed, 3*embed] tensor,
so self-attention runs a single QKV GEMM whose output the flash kernel reads in place through
strided tensor maps, and the backward kernel writes dQ|dK|dV into one packed buffer that feeds
a single weight-gradient GEMM.  The per-projection tensors stay addressable (and keep the
reference's [in, out] layout) for checkpoints.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import _backend as B
from .. import autograd
from ..tensor import Tensor
from .linear import Linear, write_param_grad
from .module import Module, compute_view


class _SlicedLinear(Linear):
    """Bias-free Linear whose weight is columns [lo, hi) of a fused parameter."""

    def __init__(self, base: Tensor, lo: int, hi: int):
        self.in_features = base._t.shape[0]
        self.out_features = hi - lo
        self.use_bias = False
        self.bias = None
        w = Tensor(_data=base._t[:, lo:hi])
        w.requires_grad = True
        w._node = autograd.Node(w, "leaf", [])
        w._base = base
        w._base_slice = (lo, hi)
        self.weight = w


class MultiHeadAttention(Module):
    causal_default = False

    def __init__(self, embed_dim: int, num_heads: int, causal: Optional[bool] = None):
        assert embed_dim % num_heads == 0, "embed_dim must be divisible by num_heads"
        self.embed_dim = embed_dim
        self.num_heads = num_heads
        self.head_dim = embed_dim // num_heads
        self.causal = self.causal_default if causal is None else bool(causal)
        self.scale = 1.0 / math.sqrt(self.head_dim)
        E = embed_dim
        fused = Tensor([E, 3 * E]).randn()
        fused._t.mul_(math.sqrt(2.0 / E))
        autograd.watch(fused)
        self.qkv_weight = fused
        self.q_proj = _SlicedLinear(fused, 0, E)
        self.k_proj = _SlicedLinear(fused, E, 2 * E)
        self.v_proj = _SlicedLinear(fused, 2 * E, 3 * E)
        self.out_proj = Linear(E, E, True)

    # ------------------------------------------------------------------ forward
    def forward(self, query: Tensor, key: Optional[Tensor] = None, value: Optional[Tensor] = None,
                seq_len: Optional[int] = None, residual: Optional[Tensor] = None) -> Tensor:
        self_attn = (key is None or key is query) and (value is None or value is query)
        total = query.shape[0]
        seq_len = seq_len or total
        batch = total // seq_len
        H, D, E = self.num_heads, self.head_dim, self.embed_dim
        x = query._t
        fused_ok = self_attn and x.is_cuda and (x.dtype == torch.bfloat16 or
                                                self.qkv_weight._compute is not None)
        if fused_ok:
            ctx_t = self._attend_fused(query, batch, seq_len)
        else:
            key = key if key is not None else query
            value = value if value is not None else query
            q = self.q_proj(query)
            k = self.k_proj(key)
            v = self.v_proj(value)
            ctx_t = self._attend(q, k, v, batch, seq_len)
        return self.out_proj(ctx_t, residual=residual)

    def _attend(self, q: Tensor, k: Tensor, v: Tensor, batch: int, seq_len: int) -> Tensor:
        H, D = self.num_heads, self.head_dim
        q4, k4, v4 = (t._t.reshape(batch, seq_len, H, D) for t in (q, k, v))
        causal, scale = self.causal, self.scale
        o, ctx = B.attention_forward(q4, k4, v4, causal, scale)
        out = Tensor(_data=o.reshape(batch * seq_len, H * D).to(q._t.dtype))

        def grad_fn(g):
            d_o = g._t.reshape(batch, seq_len, H, D)
            dq, dk, dv = B.attention_backward(q4, k4, v4, o, ctx, d_o, causal, scale)
            for t, d in ((q, dq), (k, dk), (v, dv)):
                if t.requires_grad:
                    autograd.acc_grad(t, d.reshape(batch * seq_len, H * D).to(t._t.dtype))

        autograd.record("attention", [q, k, v], out, grad_fn)
        return out

    def _attend_fused(self, x_in: Tensor, batch: int, seq_len: int) -> Tensor:
        """Self-attention on CUDA: one QKV GEMM, flash kernel on the strided result."""
        H, D, E = self.num_heads, self.head_dim, self.embed_dim
        x = x_in._t
        if x.dtype != torch.bfloat16:
            x = B.cast(x, torch.bfloat16)
        w = compute_view(self.qkv_weight, x)
        qkv = B.gemm(x, w)                                   # [B*S, 3E]
        q5 = qkv.view(batch, seq_len, 3, H, D)
        q4, k4, v4 = q5[:, :, 0], q5[:, :, 1], q5[:, :, 2]
        causal, scale = self.causal, self.scale
        o, ctx = B.attention_forward(q4, k4, v4, causal, scale)
        out = Tensor(_data=o.reshape(batch * seq_len, E))
        fused = self.qkv_weight
        parts = [self.q_proj.weight, self.k_proj.weight, self.v_proj.weight]

        def grad_fn(g):
            d_o = g._t.reshape(batch, seq_len, H, D)
            dqkv = torch.empty((batch, seq_len, 3, H, D), device=x.device, dtype=torch.bfloat16)
            B.attention_backward(q4, k4, v4, o, ctx, d_o, causal, scale, packed_out=dqkv)
            d2 = dqkv.view(batch * seq_len, 3 * E)
            if parts[0].grad is None:
                fused.grad = None   # the slices were zeroed: start a fresh accumulation
            if x_in.requires_grad:
                autograd.acc_grad(x_in, B.gemm(d2, w, b_t=True))
            write_param_grad(fused, lambda o_, acc: B.gemm(x, d2, a_t=True, out=o_, accumulate=acc))
            _propagate_fused_grad(fused, parts)

        autograd.record("self_attention", [x_in, fused] + parts, out, grad_fn)
        return out

    # ------------------------------------------------------------------ protocol
    def children(self):
        return [self.q_proj, self.k_proj, self.v_proj, self.out_proj]

    def parameters(self):
        return [self.q_proj.weight, self.k_proj.weight, self.v_proj.weight,
                self.out_proj.weight, self.out_proj.bias]

    def _moved(self):
        # the slices must keep aliasing the fused tensor after a device move
        f = self.qkv_weight
        dev = self.out_proj.weight._t.device
        if f._t.device != dev:
            f._t = f._t.to(dev)
        E = self.embed_dim
        for i, lin in enumerate((self.q_proj, self.k_proj, self.v_proj)):
            lin.weight._t = f._t[:, i * E:(i + 1) * E]

    def __repr__(self):
        return "%s(embed=%d, heads=%d%s)" % (self.__class__.__name__, self.embed_dim,
                                             self.num_heads, ", causal" if self.causal else "")


def _propagate_fused_grad(fused: Tensor, parts) -> None:
    """Expose the fused gradient through the per-projection parameters (views of it)."""
    g = fused.grad._t if fused.grad is not None else None
    if g is None:
        return
    for p in parts:
        lo, hi = p._base_slice
        if p._grad_buf is None:
            p.grad = Tensor(_data=g[:, lo:hi])
        elif p.grad is None:
            p.grad = Tensor(_data=p._grad_buf)


class FlashMultiHeadAttention(MultiHeadAttention):
    causal_default = True

    def __init__(self, embed_dim: int, num_heads: int, causal: Optional[bool] = True):
        super().__init__(embed_dim, num_heads, True if causal is None else causal)
