"""Sequential container (lua/luatorch/nn/sequential.lua): chain of layers, flattened
`parameters()`, `add`, `num_params`, printable tree."""
from __future__ import annotations

from .module import Module


class Sequential(Module):
    def __init__(self, *layers):
        self.layers = list(layers)

    def add(self, layer):
        self.layers.append(layer)
        return self

    def forward(self, input):
        out = input
        for layer in self.layers:
            out = layer(out)
        return out

    def children(self):
        return self.layers

    def parameters(self):
        params = []
        for layer in self.layers:
            params.extend(layer.parameters())
        return params

    def __repr__(self):
        lines = ["Sequential("]
        for i, layer in enumerate(self.layers):
            lines.append("  (%d): %r" % (i + 1, layer))
        lines.append(")")
        return "\n".join(lines)
