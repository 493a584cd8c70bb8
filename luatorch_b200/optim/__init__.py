"""Optimizers and LR schedulers, the `lf.optim` namespace of the reference
(lua/luatorch/init.lua:12-19)."""
from .adam import Adam, AdamW
from .scheduler import CosineAnnealing, StepLR, WarmupScheduler
from .sgd import SGD

__all__ = ["Adam", "AdamW", "SGD", "CosineAnnealing", "WarmupScheduler", "StepLR"]
