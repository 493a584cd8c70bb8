"""`lf.cuda`: AMP helpers (lua/luatorch/init.lua:41-47)."""
from . import amp
from .amp import GradScaler, autocast_bf16

__all__ = ["amp", "GradScaler", "autocast_bf16"]
