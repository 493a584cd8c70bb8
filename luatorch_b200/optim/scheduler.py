"""Learning-rate schedulers (lua/luatorch/optim/scheduler.lua): CosineAnnealing,
WarmupScheduler and StepLR.  Each mutates `optimizer.lr`; `step()` returns the new rate."""
from __future__ import annotations

import math


class CosineAnnealing:
    @classmethod
    def new(cls, *args, **kwargs):
        """`X.new(...)` is `X(...)`, the reference's constructor spelling."""
        return cls(*args, **kwargs)

    def __init__(self, optimizer, T_max: int, min_lr: float = 0.0):
        self.optimizer = optimizer
        self.T_max = T_max
        self.min_lr = min_lr or 0.0
        self.max_lr = optimizer.lr
        self.step_num = 0

    def step(self) -> float:
        self.step_num += 1
        t = min(self.step_num, self.T_max)
        lr = self.min_lr + 0.5 * (self.max_lr - self.min_lr) * (1.0 + math.cos(math.pi * t / self.T_max))
        self.optimizer.lr = lr
        return lr

    def get_lr(self) -> float:
        return self.optimizer.lr

    def state_dict(self):
        return {"step_num": self.step_num, "max_lr": self.max_lr}

    def load_state_dict(self, s):
        self.step_num, self.max_lr = int(s["step_num"]), float(s["max_lr"])

    def __repr__(self):
        return "CosineAnnealing(T=%d, min=%.6f, max=%.6f, step=%d)" % (
            self.T_max, self.min_lr, self.max_lr, self.step_num)


class WarmupScheduler:
    @classmethod
    def new(cls, *args, **kwargs):
        """`X.new(...)` is `X(...)`, the reference's constructor spelling."""
        return cls(*args, **kwargs)

    def __init__(self, optimizer, warmup_steps: int, after_scheduler=None):
        self.optimizer = optimizer
        self.warmup_steps = warmup_steps
        self.target_lr = optimizer.lr
        self.after_scheduler = after_scheduler
        self.step_num = 0

    def step(self) -> float:
        self.step_num += 1
        if self.step_num <= self.warmup_steps:
            lr = self.target_lr * (self.step_num / self.warmup_steps)
            self.optimizer.lr = lr
            return lr
        if self.after_scheduler is not None:
            return self.after_scheduler.step()
        return self.optimizer.lr

    def get_lr(self) -> float:
        return self.optimizer.lr

    def state_dict(self):
        return {"step_num": self.step_num, "target_lr": self.target_lr,
                "after": self.after_scheduler.state_dict() if self.after_scheduler else None}

    def load_state_dict(self, s):
        self.step_num, self.target_lr = int(s["step_num"]), float(s["target_lr"])
        if self.after_scheduler is not None and s.get("after") is not None:
            self.after_scheduler.load_state_dict(s["after"])

    def __repr__(self):
        return "WarmupScheduler(warmup=%d, step=%d)" % (self.warmup_steps, self.step_num)


class StepLR:
    @classmethod
    def new(cls, *args, **kwargs):
        """`X.new(...)` is `X(...)`, the reference's constructor spelling."""
        return cls(*args, **kwargs)

    def __init__(self, optimizer, step_size: int, gamma: float = 0.1):
        self.optimizer = optimizer
        self.step_size = step_size
        self.gamma = 0.1 if gamma is None else gamma
        self.base_lr = optimizer.lr
        self.epoch = 0

    def step(self) -> float:
        self.epoch += 1
        lr = self.base_lr * (self.gamma ** (self.epoch // self.step_size))
        self.optimizer.lr = lr
        return lr

    def get_lr(self) -> float:
        return self.optimizer.lr

    def state_dict(self):
        return {"epoch": self.epoch, "base_lr": self.base_lr}

    def load_state_dict(self, s):
        self.epoch, self.base_lr = int(s["epoch"]), float(s["base_lr"])

    def __repr__(self):
        return "StepLR(step_size=%d, gamma=%.4f, epoch=%d)" % (self.step_size, self.gamma, self.epoch)
