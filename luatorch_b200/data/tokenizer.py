"""Character-level tokenizer (lua/luatorch/data/tokenizer.lua): sorted unique bytes of the
training text map to 0-based ids; `save` writes the vocabulary size on the first line then one
`id byte` pair per line, and `Tokenizer.load` reads that format back."""
from __future__ import annotations

from typing import List

import torch

from ..tensor import Tensor


class Tokenizer:
    def __init__(self, text=""):
        data = text.encode("latin-1", "replace") if isinstance(text, str) else bytes(text)
        chars = sorted(set(data))
        self.char_to_id = {c: i for i, c in enumerate(chars)}
        self.id_to_char = {i: c for i, c in enumerate(chars)}
        self.vocab_size = len(chars)

    @classmethod
    def new(cls, text=""):
        return cls(text)

    def _bytes(self, text) -> bytes:
        return text.encode("latin-1", "replace") if isinstance(text, str) else bytes(text)

    def encode(self, text) -> List[int]:
        ids = []
        for c in self._bytes(text):
            i = self.char_to_id.get(c)
            if i is None:
                raise ValueError("luatorch error: unknown character: %r" % chr(c))
            ids.append(i)
        return ids

    def encode_tensor(self, text) -> Tensor:
        return Tensor(_data=torch.tensor(self.encode(text), dtype=torch.float32))

    def decode(self, ids) -> str:
        out = bytearray()
        for i in ids:
            c = self.id_to_char.get(int(i))
            if c is None:
                raise ValueError("luatorch error: unknown token id: %s" % i)
            out.append(c)
        return out.decode("latin-1")

    def decode_tensor(self, tensor: Tensor) -> str:
        return self.decode(int(v) for v in tensor._t.reshape(-1).tolist())

    def save(self, path: str) -> None:
        with open(path, "w") as f:
            f.write("%d\n" % self.vocab_size)
            for i in range(self.vocab_size):
                f.write("%d %d\n" % (i, self.id_to_char[i]))

    @classmethod
    def load(cls, path: str) -> "Tokenizer":
        self = cls.__new__(cls)
        self.char_to_id, self.id_to_char = {}, {}
        with open(path) as f:
            self.vocab_size = int(f.readline())
            for _ in range(self.vocab_size):
                i, b = f.readline().split()
                self.char_to_id[int(b)] = int(i)
                self.id_to_char[int(i)] = int(b)
        return self

    def __repr__(self):
        return "Tokenizer(vocab_size=%d)" % self.vocab_size
