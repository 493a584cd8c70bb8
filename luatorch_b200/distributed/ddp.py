"""Data-parallel training wrapper.

`DDP(model, num_gpus)` keeps the reference's surface (lua/luatorch/distributed/ddp.lua):
`forward` / call, `sync_gradients()`, `parameters()`, `zero_grad()`, `num_params()`,
`train()` / `eval()`.  The reference wrapper is a stub: it never replicates the model or
splits the batch and all-reduces one gradient pointer against itself, one blocking NCCL call
per parameter (ddp.lua:48-61).  This one is real:

  * one rank per GPU, identical replicas (rank 0's weights are broadcast at construction),
    every rank feeds its own micro-batch;
  * parameters live in a flat arena (fp32 master, bf16 shadow, bf16 gradients); the gradient
    and shadow arenas are peer-mapped on every rank;
  * the arena is cut into buckets in reverse parameter order; when backward has produced the
    last gradient of a bucket, ONE kernel on a side stream reduces the bucket over NVLink,
    scales by 1/world, applies AdamW and publishes the updated bf16 weights, overlapping the
    rest of backward.  `mode`:
        "sharded"    two-shot: rank r reduces slice r of the bucket, updates slice r of
                     master / m / v and stores the new bf16 weights into every rank's shadow
                     arena (reduce-scatter + shard AdamW + all-gather in one launch);
        "replicated" one-shot: every rank reduces the whole bucket and updates its full
                     replica (least latency; meant for small models);
        "nccl"       baseline: process-group all_reduce per bucket, then the flat AdamW launch.
  * `optimizer.step()` after `sync_gradients()` keeps working: once an optimizer is attached
    its `step` only finalises the fused update (joins the side stream, advances the counter).

Every device-side wait is bounded; `check()` surfaces a timed-out wait as `CommError`.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from .. import _backend as B
from ..parallel.arena import ParamArena
from ..tensor import Tensor
from . import comm


class DDP:
    @classmethod
    def new(cls, *args, **kwargs):
        """`X.new(...)` is `X(...)`, the reference's constructor spelling."""
        return cls(*args, **kwargs)

    def __init__(self, model, num_gpus: Optional[int] = None, bucket_mb: float = 32.0,
                 mode: str = "sharded", device: Optional[str] = None, max_blocks: int = 0,
                 broadcast_init: bool = True):
        comm.init(num_gpus)
        self.model = model
        self.world = comm.world_size()
        self.rank = comm.rank()
        self.num_gpus = self.world
        self.mode = mode
        self.max_blocks = max_blocks
        self.device = device or ("cuda" if torch.cuda.is_available() else "cpu")
        self.optimizer = None
        self._step_check = 0
        on_gpu = self.device == "cuda"
        if on_gpu:
            model.cuda()
        # arenas: gradients and bf16 shadow weights in peer-mapped memory when possible
        self._bufs = {}

        def allocator(n, dtype):
            if not on_gpu:
                return torch.zeros(n, dtype=dtype)
            esz = torch.empty((), dtype=dtype).element_size()
            buf = comm.SymmetricBuffer(n * esz)
            self._bufs[len(self._bufs)] = buf
            return buf.typed(dtype)[:n]

        self.arena = ParamArena(model.parameters(), device=self.device,
                                compute_dtype=torch.bfloat16 if on_gpu else None,
                                grad_dtype=torch.bfloat16 if on_gpu else torch.float32,
                                allocator=allocator)
        if on_gpu:
            self.shadow_buf = self._bufs[0]
            self.grad_buf = self._bufs[1]
            self.peer = self.world > 1 and self.grad_buf.peer_mapped and self.shadow_buf.peer_mapped
        else:
            self.shadow_buf = self.grad_buf = None
            self.peer = False
        if self.world > 1 and self.mode != "nccl" and not self.peer:
            self.mode = "nccl"   # no peer mapping on this machine: process-group collectives
        bucket_elems = max(2048, int(bucket_mb * 1024 * 1024 / 2))
        self.buckets = self.arena.buckets(bucket_elems)
        self._unit_bucket = {}
        for bi, b in enumerate(self.buckets):
            for u in b["units"]:
                self._unit_bucket.setdefault(id(u), []).append(bi)
        self._pending = [0] * len(self.buckets)
        self._launched = [False] * len(self.buckets)
        self._cursor = 0
        self._comm_stream = torch.cuda.Stream() if on_gpu else None
        for u in self.arena.units:
            u._hook = self._on_grad_ready
        if broadcast_init and self.world > 1:
            self._broadcast_parameters()
        self._reset_step()
        if self.rank == 0:
            print("DDP: model replicated across %d gpus (%s, %d buckets)" % (
                self.world, self.mode, len(self.buckets)))

    # ------------------------------------------------------------------ reference surface
    def forward(self, *args, **kwargs):
        return self.model.forward(*args, **kwargs)

    __call__ = forward

    def parameters(self) -> List[Tensor]:
        return self.model.parameters()

    def zero_grad(self) -> None:
        self.arena.zero_grad()
        self._reset_step()

    def num_params(self) -> int:
        return self.model.num_params() if hasattr(self.model, "num_params") else 0

    def train(self):
        if hasattr(self.model, "train"):
            self.model.train()

    def eval(self):
        if hasattr(self.model, "eval"):
            self.model.eval()

    def __repr__(self):
        return "DDP(gpus=%d, mode=%s, model=%r)" % (self.world, self.mode, self.model)

    # ------------------------------------------------------------------ setup helpers
    def _broadcast_parameters(self) -> None:
        a = self.arena
        if self.peer:
            # rank 0's fp32 master goes out in pieces staged through the peer-mapped gradient
            # arena (it holds total/2 floats), copied by the peer_broadcast kernel
            stage = self.grad_buf.typed(torch.float32)
            cap = stage.numel()
            for lo in range(0, a.total, cap):
                hi = min(a.total, lo + cap)
                piece = a.master[lo:hi]
                comm.broadcast_(piece, 0, self.grad_buf)
            self.grad_buf.data.zero_()
        else:
            dist.broadcast(a.master, src=0)
        a.sync_shadow()
        if self.device == "cuda":
            torch.cuda.synchronize()
        comm.barrier()

    def attach(self, optimizer) -> None:
        """Fuse `optimizer` (Adam / AdamW over this wrapper's parameters) into the gradient
        reduction.  Its `step()` becomes the join point of the fused update."""
        if optimizer.arena is not self.arena:
            raise ValueError("optimizer must be built from ddp.parameters() after wrapping")
        self.optimizer = optimizer
        optimizer._ddp = self
        optimizer._plain_step = optimizer.step
        optimizer.step = self._optimizer_step

    # ------------------------------------------------------------------ per-step machinery
    def _reset_step(self) -> None:
        for bi, b in enumerate(self.buckets):
            self._pending[bi] = len(b["units"])
            self._launched[bi] = False
        self._cursor = 0
        self._synced = False
        self._comm_used = False      # did this step put work on the communication stream?

    def _on_grad_ready(self, unit: Tensor) -> None:
        for bi in self._unit_bucket.get(id(unit), ()):
            self._pending[bi] -= 1
        self._launch_ready()

    def _launch_ready(self, force: bool = False) -> None:
        # buckets go out strictly in index order so every rank issues the same sequence
        while self._cursor < len(self.buckets) and (force or self._pending[self._cursor] <= 0):
            self._launch_bucket(self._cursor)
            self._cursor += 1

    def _fusable(self) -> bool:
        return (self.optimizer is not None and self.device == "cuda" and
                hasattr(self.optimizer, "beta1"))

    def _launch_bucket(self, bi: int) -> None:
        if self._launched[bi]:
            return
        self._launched[bi] = True
        if self.world == 1 and not self._fusable():
            return
        b = self.buckets[bi]
        lo, hi = b["start"], b["end"]
        a = self.arena
        if self.device != "cuda":
            if self.world > 1:
                dist.all_reduce(a.grad[lo:hi], op=dist.ReduceOp.SUM)
                a.grad[lo:hi].div_(self.world)
            return
        cur = torch.cuda.current_stream()
        ev = torch.cuda.Event()
        ev.record(cur)
        self._comm_stream.wait_event(ev)
        self._comm_used = True
        with torch.cuda.stream(self._comm_stream):
            opt = self.optimizer
            if self._fusable() and (self.world == 1 or self.mode in ("sharded", "replicated")):
                t = opt.t + 1
                bc1, bc2 = 1.0 - opt.beta1 ** t, 1.0 - opt.beta2 ** t
                seg_end, seg_wd = opt.segments()
                if self.world == 1:
                    B.adamw_flat(a.master[lo:hi], a.shadow[lo:hi], a.grad[lo:hi],
                                 opt.m_flat[lo:hi], opt.v_flat[lo:hi],
                                 (seg_end - lo).clamp_(min=0), seg_wd, opt.lr, opt.beta1,
                                 opt.beta2, opt.epsilon, bc1, bc2, opt.grad_scale,
                                 opt.skip_flag)
                else:
                    B.ext().allreduce_adamw(
                        self.grad_buf.ptrs, self.grad_buf.signal_ptrs, self.rank, self.world, lo,
                        hi - lo, a.master, self.shadow_buf.ptrs, opt.m_flat, opt.v_flat, seg_end,
                        seg_wd, opt.lr, opt.beta1, opt.beta2, opt.epsilon, bc1, bc2,
                        opt.grad_scale / self.world, comm.next_epoch(),
                        1 if self.mode == "sharded" else 0, self.max_blocks, comm.status_buffer())
            elif self.world > 1:
                if self.mode == "nccl" or not self.peer:
                    g = a.grad[lo:hi]
                    dist.all_reduce(g, op=dist.ReduceOp.SUM)
                    B.scalar_inplace("mul", g, 1.0 / self.world)
                else:
                    B.ext().peer_allreduce(self.grad_buf.ptrs, self.grad_buf.signal_ptrs,
                                           self.rank, self.world, lo, hi - lo, 1, 1.0 / self.world,
                                           comm.next_epoch(), comm.status_buffer())

    def sync_gradients(self) -> None:
        """Make sure every bucket has been issued and the compute stream waits for them."""
        if self._synced:
            return
        self._launch_ready(force=True)
        # join the communication stream only if this step forked onto it (a stream that did no
        # work must not be waited on from a stream that is being captured into a graph)
        if self.device == "cuda" and self._comm_used:
            ev = torch.cuda.Event()
            ev.record(self._comm_stream)
            torch.cuda.current_stream().wait_event(ev)
        self._synced = True

    def _optimizer_step(self) -> None:
        opt = self.optimizer
        self.sync_gradients()
        fused = self._fusable() and (self.world == 1 or self.mode in ("sharded", "replicated"))
        if fused:
            opt.t += 1
        else:
            opt._plain_step()
        self._step_check += 1

    def check(self) -> None:
        """Surface device-side communication errors (one small device-to-host read)."""
        if self.device == "cuda":
            comm.check_status()

    def gather_master(self) -> None:
        """In "sharded" mode each rank owns the fp32 master of its bucket slices only; this
        refreshes the other slices from their owners (before writing a checkpoint)."""
        if self.world == 1 or self.mode != "sharded":
            return
        a = self.arena
        for b in self.buckets:
            lo, hi = b["start"], b["end"]
            span = (hi - lo) // self.world
            parts = [torch.empty(span, device=a.master.device, dtype=torch.float32)
                     for _ in range(self.world)]
            dist.all_gather(parts, a.master[lo + self.rank * span: lo + (self.rank + 1) * span].contiguous())
            for r, p in enumerate(parts):
                a.master[lo + r * span: lo + (r + 1) * span].copy_(p)
