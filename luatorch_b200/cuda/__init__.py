"""`lf.cuda`: AMP helpers (lua/luatorch/init.lua:41-47), CUDA-graph replay of a step and the
one-step-behind reader for per-step device scalars."""
from . import amp, fetch, graph
from .amp import GradScaler, autocast_bf16
from .fetch import ScalarFetcher
from .graph import GraphedStep

__all__ = ["amp", "fetch", "graph", "GradScaler", "autocast_bf16", "GraphedStep", "ScalarFetcher"]
