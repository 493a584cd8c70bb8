"""Multi-layer perceptron (lua/luatorch/models/mlp.lua): `MLP([784, 256, 128, 10])` builds
Linear layers with ReLU between them (none after the last) inside a Sequential.  On CUDA in
bf16 each hidden layer is one GEMM with bias + ReLU in the epilogue."""
from __future__ import annotations

from typing import Sequence

from ..nn.activation import ReLU
from ..nn.linear import Linear
from ..nn.module import Module
from ..nn.sequential import Sequential


class MLP(Module):
    def __init__(self, sizes: Sequence[int]):
        self.sizes = list(sizes)
        layers = []
        for i in range(len(self.sizes) - 1):
            layers.append(Linear(self.sizes[i], self.sizes[i + 1]))
            if i < len(self.sizes) - 2:
                layers.append(ReLU())
        self.net = Sequential(*layers)

    def forward(self, input):
        return self.net(input)

    def children(self):
        return [self.net]

    def parameters(self):
        return self.net.parameters()

    def __repr__(self):
        return "MLP(%s)" % " -> ".join(str(s) for s in self.sizes)
