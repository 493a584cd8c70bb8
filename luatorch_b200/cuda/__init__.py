"""`lf.cuda`: AMP helpers (lua/luatorch/init.lua:41-47) and CUDA-graph replay of a step."""
from . import amp, graph
from .amp import GradScaler, autocast_bf16
from .graph import GraphedStep

__all__ = ["amp", "graph", "GradScaler", "autocast_bf16", "GraphedStep"]
