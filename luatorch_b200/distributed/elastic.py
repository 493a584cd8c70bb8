"""Failure detection and restart support (the reference has none: errors are printed and
surface as nil / -1, csrc/distributed/nccl_wrapper.cu:12-19).

Host side only, so it is testable with CPU ranks and never needs a GPU fault:

  * `Heartbeat`: every rank publishes a counter in the job's key-value store from a
    background thread; `check()` raises `RankFailure` naming the ranks whose counter stopped
    advancing, so the survivors learn of a lost rank BEFORE they enter the next collective.
  * `run_step_guarded`: runs one training step and converts a collective timeout /
    `CommError` / `RankFailure` into a `StepFailed` carrying the last good step.
  * `resume`: reload the last checkpoint (+ training-state sidecars) into a freshly built
    model / optimizer, possibly with a different world size; bucket boundaries are a pure
    function of the parameter list, so re-bucketing is deterministic.
The device side of failure detection is the bounded wait in every collective kernel
(csrc/comm/comm_kernels.cu) reported through `comm.check_status()`.
"""
from __future__ import annotations

import threading
import time
from typing import Callable, List, Optional

from . import comm


class RankFailure(RuntimeError):
    def __init__(self, ranks: List[int]):
        self.ranks = ranks
        super().__init__("ranks stopped responding: %s" % ranks)


class StepFailed(RuntimeError):
    def __init__(self, step: int, cause: BaseException):
        self.step, self.cause = step, cause
        super().__init__("training step %d failed: %r" % (step, cause))


class Heartbeat:
    def __init__(self, store, rank: int, world: int, interval_s: float = 0.2,
                 stale_after_s: float = 2.0, prefix: str = "lt_hb"):
        self.store, self.rank, self.world = store, rank, world
        self.interval_s, self.stale_after_s, self.prefix = interval_s, stale_after_s, prefix
        self._stop = threading.Event()
        self._count = 0
        self._last_seen = {}
        self._thread = threading.Thread(target=self._beat, daemon=True)
        self._beat_once()
        self._thread.start()

    def _key(self, r: int) -> str:
        return "%s/%d" % (self.prefix, r)

    def _beat_once(self):
        self._count += 1
        self.store.set(self._key(self.rank), str(self._count))

    def _beat(self):
        while not self._stop.wait(self.interval_s):
            try:
                self._beat_once()
            except Exception:
                return

    def stop(self):
        self._stop.set()
        self._thread.join(timeout=2.0)

    def check(self) -> None:
        now = time.monotonic()
        dead = []
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                v = int(self.store.get(self._key(r)))
            except Exception:
                v = -1
            prev = self._last_seen.get(r)
            if prev is None or prev[0] != v:
                self._last_seen[r] = (v, now)
            elif now - prev[1] > self.stale_after_s:
                dead.append(r)
        if dead:
            raise RankFailure(dead)


def run_step_guarded(step_fn: Callable[[], object], step: int,
                     heartbeat: Optional[Heartbeat] = None):
    """Run `step_fn()`; peers are checked on the host first so a lost rank is reported
    without entering a collective that could never complete."""
    try:
        if heartbeat is not None:
            heartbeat.check()
        out = step_fn()
        comm.check_status() if comm._state.get("status") is not None else None
        return out
    except (RankFailure, comm.CommError, RuntimeError) as e:
        raise StepFailed(step, e)


def resume(build_fn: Callable[[], tuple], checkpoint_path: str):
    """`build_fn()` -> (model, optimizer, scheduler, scaler) for the CURRENT world size; loads
    parameters and training state saved by `io.checkpoint.save` / `save_training_state`."""
    from ..io import checkpoint
    model, optimizer, scheduler, scaler = build_fn()
    if hasattr(model, "load_checkpoint"):
        # the data-parallel wrapper restores sharded master weights and moments itself
        meta = model.load_checkpoint(checkpoint_path, optimizer, scheduler, scaler)
        return model, optimizer, scheduler, scaler, meta
    inner = getattr(model, "model", model)
    checkpoint.load(inner, checkpoint_path)
    arena = getattr(model, "arena", None)
    if arena is not None:
        arena.sync_shadow()
    meta = checkpoint.load_training_state(checkpoint_path, inner, optimizer, scheduler, scaler)
    return model, optimizer, scheduler, scaler, meta
