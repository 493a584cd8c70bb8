"""Pre-LayerNorm transformer block (lua/luatorch/nn/transformer.lua:29-144):

    x = x + drop(attn(ln1(x)))
    x = x + drop(ffn2(gelu(ffn1(ln2(x)))))

ffn_mult 4, dropout 0.1, causal flash attention by default; parameter order
ln1, attn, ln2, ffn1, ffn2.  `forward(x, seq_len)` takes the flattened [batch*seq_len, embed]
activations; `seq_len` separates the sequences (the reference drops it, so a batch is
attended as one long sequence, and its residual adds bypass the tape so no gradient crosses a
block; both are fixed here).

On CUDA in bf16 a block is 5 GEMMs + flash attention + 2 LayerNorms forward: bias, GELU and
both residual adds run in GEMM epilogues, and in backward the LayerNorm kernels absorb the
residual-gradient adds.
"""
from __future__ import annotations

from typing import Optional

from .. import autograd
from ..tensor import Tensor
from .activation import GELU
from .dropout import Dropout
from .layernorm import LayerNorm
from .linear import Linear
from .module import Module
from .multihead import FlashMultiHeadAttention, MultiHeadAttention


class TransformerBlock(Module):
    def __init__(self, embed_dim: int, num_heads: int, dropout_p: Optional[float] = 0.1,
                 ffn_mult: Optional[int] = 4, use_flash: Optional[bool] = True):
        dropout_p = 0.1 if dropout_p is None else dropout_p
        ffn_mult = ffn_mult or 4
        use_flash = True if use_flash is None else use_flash
        self.embed_dim = embed_dim
        ffn_dim = embed_dim * ffn_mult
        self.ln1 = LayerNorm(embed_dim)
        self.attn = (FlashMultiHeadAttention(embed_dim, num_heads, True) if use_flash
                     else MultiHeadAttention(embed_dim, num_heads))
        self.drop1 = Dropout(dropout_p)
        self.ln2 = LayerNorm(embed_dim)
        self.ffn1 = Linear(embed_dim, ffn_dim)
        self.gelu = GELU()
        self.ffn2 = Linear(ffn_dim, embed_dim)
        self.drop2 = Dropout(dropout_p)
        self.training = True

    def forward(self, x: Tensor, seq_len: Optional[int] = None) -> Tensor:
        fuse1 = not (self.training and self.drop1.p > 0.0)
        fuse2 = not (self.training and self.drop2.p > 0.0)
        normed = self.ln1(x)
        if fuse1:
            x = self.attn(normed, seq_len=seq_len, residual=x)
        else:
            x = autograd.add(x, self.drop1(self.attn(normed, seq_len=seq_len)))
        normed = self.ln2(x)
        h = self.ffn1(normed, act="gelu")
        if fuse2:
            x = self.ffn2(h, residual=x, sole_consumer=True)
        else:
            x = autograd.add(x, self.drop2(self.ffn2(h, sole_consumer=True)))
        return x

    def children(self):
        return [self.ln1, self.attn, self.drop1, self.ln2, self.ffn1, self.ffn2, self.drop2]

    def parameters(self):
        params = []
        for layer in (self.ln1, self.attn, self.ln2, self.ffn1, self.ffn2):
            params.extend(layer.parameters())
        return params

    def __repr__(self):
        return "TransformerBlock(embed=%d, attn=%r)" % (self.embed_dim, self.attn)
