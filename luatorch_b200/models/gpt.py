"""GPT decoder (lua/luatorch/models/gpt.lua).

`GPT(vocab_size, embed_dim, num_heads, num_layers, max_seq_len, dropout=0.1)`: token
embedding + positional encoding + embedding dropout + N pre-LN transformer blocks + final
LayerNorm + UNTIED head Linear(embed, vocab, bias=False).  `forward(input[B, S])` returns
logits [B*S, vocab]; `generate(prompt, max_tokens, temperature, top_k)` samples with a full
re-forward per token, context cropped to `max_seq_len`; `parameters()` order is token_emb,
positional (if learned), blocks, final_ln, head; `no_decay_params()` is every LayerNorm
parameter plus the ffn1 / ffn2 / out_proj biases.

Extension: `pos="learned"` selects a LearnedPE table (the reference always uses the fixed
sinusoidal table).  On CUDA the token gather and the positional add are one kernel, and the
head weight is stored with its row padded to a multiple of 8 columns so TMA can address the
50257-wide vocabulary (checkpoints still hold the unpadded [embed, vocab] matrix).
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch

from .. import _backend as B
from ..utils import debug as _debug
from .. import autograd
from ..nn.dropout import Dropout
from ..nn.embedding import Embedding, embedding_backward_into
from ..nn.layernorm import LayerNorm
from ..nn.linear import Linear
from ..nn.module import Module
from ..nn.positional import LearnedPE, SinusoidalPE, positional_backward_into
from ..nn.transformer import TransformerBlock
from ..tensor import Tensor


class GPT(Module):
    def __init__(self, vocab_size: int, embed_dim: int, num_heads: int, num_layers: int,
                 max_seq_len: int, dropout: Optional[float] = 0.1, pos: str = "sinusoidal"):
        dropout = 0.1 if dropout is None else dropout
        self.vocab_size = vocab_size
        self.embed_dim = embed_dim
        self.num_heads = num_heads
        self.num_layers = num_layers
        self.max_seq_len = max_seq_len
        self.token_emb = Embedding(vocab_size, embed_dim)
        self.pos_enc = (LearnedPE(max_seq_len, embed_dim) if pos == "learned"
                        else SinusoidalPE(max_seq_len, embed_dim))
        self.emb_drop = Dropout(dropout)
        self.blocks: List[TransformerBlock] = [
            TransformerBlock(embed_dim, num_heads, dropout) for _ in range(num_layers)]
        self.final_ln = LayerNorm(embed_dim)
        self.head = Linear(embed_dim, vocab_size, False, pad_out=True)
        self.training = True

    # ------------------------------------------------------------------ forward
    def _embed(self, ids: torch.Tensor, seq_len: int) -> Tensor:
        w = self.token_emb.weight
        if w._t.is_cuda:
            if not ids.is_cuda:
                ids = ids.cuda()
            ids = B._labels(ids)
            table = w._compute if w._compute is not None else w._t
            learned = isinstance(self.pos_enc, LearnedPE)
            if learned:
                pw = self.pos_enc.weight
                pos_table = pw._compute if (pw._compute is not None and
                                            pw._compute.dtype == table.dtype) else pw._t.to(table.dtype)
            else:
                pos_table = self.pos_enc._table(table)
            y, err = B.ext().embedding_forward(table, ids, pos_table, seq_len)
            _debug.check_index_word(err, "GPT token embedding: token id")
            out = Tensor(_data=y)
            batch = ids.numel() // seq_len
            pos_enc = self.pos_enc

            def grad_fn(g):
                if w.requires_grad:
                    embedding_backward_into(w, g._t, ids)
                if learned and pos_enc.weight.requires_grad:
                    positional_backward_into(pos_enc.weight, g._t, batch, seq_len)

            autograd.record("embed_tokens", [w, pos_enc.weight if learned else None], out, grad_fn)
            return out
        x = self.token_emb(Tensor(_data=ids))
        return self.pos_enc(x, seq_len)

    def forward(self, input: Tensor) -> Tensor:
        shape = input.shape
        seq_len = shape[1] if len(shape) >= 2 else shape[0]
        x = self._embed(input._t.reshape(-1), seq_len)
        x = self.emb_drop(x)
        for block in self.blocks:
            x = block(x, seq_len)
        x = self.final_ln(x)
        return self.head(x)

    # ------------------------------------------------------------------ sampling
    def generate(self, prompt: Tensor, max_tokens: int = 100, temperature: float = 1.0,
                 top_k: int = 0) -> Tensor:
        temperature = 1.0 if temperature is None else temperature
        top_k = top_k or 0
        was_training = self.training
        self.eval()
        # a Tensor of token ids (as in the reference) or any plain sequence of ints
        src = prompt._t if isinstance(prompt, Tensor) else torch.as_tensor(prompt)
        tokens = [int(v) for v in src.reshape(-1).tolist()]
        dev = self.token_emb.weight._t.device
        gen = B.cpu_generator()
        with autograd.no_grad():
            for _ in range(max_tokens or 100):
                ctx = tokens[-self.max_seq_len:]
                inp = Tensor(_data=torch.tensor(ctx, dtype=torch.float32, device=dev).reshape(1, -1))
                autograd.zero_graph()
                logits = self.forward(inp)
                last = logits._t[len(ctx) - 1, :self.vocab_size].float().cpu()
                if temperature != 1.0:
                    last = last / temperature
                if 0 < top_k < self.vocab_size:
                    thresh = torch.topk(last, top_k).values[-1]
                    last = torch.where(last < thresh, torch.full_like(last, -math.inf), last)
                probs = torch.softmax(last, 0)
                r = torch.rand((), generator=gen).item()
                idx = int(torch.searchsorted(torch.cumsum(probs, 0), torch.tensor(r)).clamp(max=self.vocab_size - 1))
                tokens.append(idx)
        if was_training:
            self.train()
        return Tensor(_data=torch.tensor(tokens, dtype=torch.float32))

    # ------------------------------------------------------------------ protocol
    def children(self):
        return [self.token_emb, self.pos_enc, self.emb_drop, *self.blocks, self.final_ln, self.head]

    def parameters(self):
        params = list(self.token_emb.parameters())
        params.extend(self.pos_enc.parameters())
        for b in self.blocks:
            params.extend(b.parameters())
        params.extend(self.final_ln.parameters())
        params.extend(self.head.parameters())
        return params

    def no_decay_params(self):
        nd = list(self.final_ln.parameters())
        for b in self.blocks:
            nd.extend(b.ln1.parameters())
            nd.extend(b.ln2.parameters())
            for lin in (b.ffn1, b.ffn2, b.attn.out_proj):
                if lin.use_bias:
                    nd.append(lin.bias)
        return nd

    def __repr__(self):
        return "GPT(vocab=%d, embed=%d, heads=%d, layers=%d, max_seq=%d, params=%d)" % (
            self.vocab_size, self.embed_dim, self.num_heads, self.num_layers, self.max_seq_len,
            self.num_params())
