"""Training logger (lua/luatorch/utils/logger.lua): running means of loss / accuracy,
a line every `print_every` steps, full history, CSV export with the header
`step,epoch,loss,accuracy,lr`.  Extensions: optional tokens-per-second column fed with
device-timed step durations, per-bucket communication time and its overlap with backward
(`log_comm`, fed from `DDP.comm_profile()`), memory-pool statistics, and a JSON-lines sink."""
from __future__ import annotations

import json
from typing import Optional


class Logger:
    def __init__(self, print_every: int = 100, jsonl_path: Optional[str] = None):
        self.print_every = print_every or 100
        self.step = 0
        self.epoch = 0
        self.history = []
        self.running_loss = 0.0
        self.running_acc = 0.0
        self.running_n = 0
        self.current_lr = 0.0
        self.running_tokens = 0
        self.running_ms = 0.0
        self._jsonl = open(jsonl_path, "a") if jsonl_path else None

    @classmethod
    def new(cls, *a, **k):
        return cls(*a, **k)

    def log(self, loss=None, accuracy=None, lr=None, tokens: int = 0, step_ms: float = 0.0):
        self.step += 1
        self.running_loss += loss or 0
        self.running_acc += accuracy or 0
        self.running_n += 1
        self.current_lr = lr or self.current_lr
        self.running_tokens += tokens
        self.running_ms += step_ms
        entry = {"step": self.step, "epoch": self.epoch, "loss": loss or 0,
                 "accuracy": accuracy or 0, "lr": self.current_lr}
        self.history.append(entry)
        if self._jsonl is not None:
            rec = dict(entry)
            if step_ms:
                rec["tokens_per_s"] = tokens / (step_ms * 1e-3)
            self._jsonl.write(json.dumps(rec) + "\n")
            self._jsonl.flush()
        if self.step % self.print_every == 0:
            self.print_summary()

    def log_comm(self, profile: dict, pool: Optional[dict] = None) -> None:
        """Record the data-parallel engine's communication profile (`DDP.comm_profile()`:
        device time of every bucket's fused reduce + optimizer kernel, their sum, and the share
        that ran under backward) and optional allocator statistics; printed with the next
        summary line and written to the JSON-lines sink."""
        self.comm = {"buckets_ms": [round(x, 4) for x in profile.get("buckets_ms", [])],
                     "total_ms": round(profile.get("total_ms", 0.0), 4),
                     "overlap": round(profile.get("overlap", 0.0), 4)}
        if pool:
            self.comm["pool"] = pool
        if self._jsonl is not None:
            self._jsonl.write(json.dumps({"step": self.step, "comm": self.comm}) + "\n")
            self._jsonl.flush()

    def set_epoch(self, epoch: int):
        self.epoch = epoch

    def print_summary(self):
        if self.running_n == 0:
            return
        avg_loss = self.running_loss / self.running_n
        avg_acc = self.running_acc / self.running_n
        parts = ["step %6d" % self.step]
        if self.epoch > 0:
            parts.append("epoch %3d" % self.epoch)
        parts.append("loss %.4f" % avg_loss)
        if avg_acc > 0:
            parts.append("acc %.2f%%" % (avg_acc * 100))
        if self.current_lr > 0:
            parts.append("lr %.2e" % self.current_lr)
        if self.running_ms > 0 and self.running_tokens > 0:
            parts.append("tok/s %.0f" % (self.running_tokens / (self.running_ms * 1e-3)))
        comm = getattr(self, "comm", None)
        if comm and comm["buckets_ms"]:
            parts.append("comm %.3f ms in %d buckets (%.0f%% under backward)" % (
                comm["total_ms"], len(comm["buckets_ms"]), 100 * comm["overlap"]))
        print("  ".join(parts))
        self.running_loss = self.running_acc = 0.0
        self.running_n = 0
        self.running_tokens, self.running_ms = 0, 0.0

    def save_csv(self, path: str):
        with open(path, "w") as f:
            f.write("step,epoch,loss,accuracy,lr\n")
            for e in self.history:
                f.write("%d,%d,%.6f,%.6f,%.8f\n" % (e["step"], e["epoch"], e["loss"], e["accuracy"], e["lr"]))

    def __repr__(self):
        return "Logger(step=%d, history=%d entries)" % (self.step, len(self.history))
