"""`lf.models`: GPT and MLP (lua/luatorch/init.lua:27-30)."""
from .gpt import GPT
from .mlp import MLP

__all__ = ["GPT", "MLP"]
