"""`lf.export`: ONNX export (lua/luatorch/init.lua:63-69)."""
from . import onnx

__all__ = ["onnx"]
