"""Character-level language-modelling dataset (lua/luatorch/data/dataset.lua): reads a text
file, builds the tokenizer from the whole text, keeps the first `split_pct` (0.9) of the
tokens for 'train' and the rest otherwise; `get(idx)` returns the window `[idx, idx+seq_len)`
and the same window shifted by one; `get_batch(n)` draws n random windows."""
from __future__ import annotations

import torch

from .. import _backend as B
from ..tensor import Tensor
from .tokenizer import Tokenizer


class TextDataset:
    def __init__(self, path: str, seq_len: int, split: str = "train", split_pct: float = 0.9,
                 verbose: bool = True):
        with open(path, "rb") as f:
            text = f.read()
        self.tokenizer = Tokenizer(text)
        self.vocab_size = self.tokenizer.vocab_size
        self.seq_len = seq_len
        lut = torch.zeros(256, dtype=torch.float32)
        for c, i in self.tokenizer.char_to_id.items():
            lut[c] = i
        all_ids = lut[torch.frombuffer(bytearray(text), dtype=torch.uint8).long()]
        split_idx = int(all_ids.numel() * (0.9 if split_pct is None else split_pct))
        ids = all_ids[:split_idx] if (split or "train") == "train" else all_ids[split_idx:]
        self.data = Tensor(_data=ids.contiguous())
        self.n_samples = ids.numel() - seq_len
        if verbose:
            print("TextDataset(%s): %d tokens, %d samples, vocab=%d" % (
                split or "train", ids.numel(), self.n_samples, self.vocab_size))

    @classmethod
    def new(cls, *a, **k):
        return cls(*a, **k)

    def get(self, idx: int):
        d = self.data._t
        return (Tensor(_data=d[idx:idx + self.seq_len].clone()),
                Tensor(_data=d[idx + 1:idx + self.seq_len + 1].clone()))

    def get_batch(self, batch_size: int):
        starts = torch.randint(0, self.n_samples, (batch_size,), generator=B.cpu_generator())
        offs = starts.unsqueeze(1) + torch.arange(self.seq_len).unsqueeze(0)
        d = self.data._t
        return Tensor(_data=d[offs]), Tensor(_data=d[offs + 1])

    def __repr__(self):
        return "TextDataset(samples=%d, seq_len=%d, vocab=%d)" % (
            self.n_samples, self.seq_len, self.vocab_size)
