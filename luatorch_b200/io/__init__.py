"""`lf.io`: checkpoint save / load (lua/luatorch/init.lua:32-34)."""
from . import checkpoint

__all__ = ["checkpoint"]
