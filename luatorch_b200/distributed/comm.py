"""Process-group bootstrap, symmetric (peer-mapped) memory and the collective entry points.

The reference's communication layer is a single-process wrapper around `ncclCommInitAll`,
`ncclAllReduce(ncclAvg)` and `ncclBroadcast` (csrc/distributed/nccl_wrapper.cu:37-135,
lua/luatorch/distributed/init.lua:16-49).  Here the process model is one rank per GPU:

  * `init()` joins the job described by RANK / WORLD_SIZE / LOCAL_RANK / MASTER_ADDR /
    MASTER_PORT (a single process with no such variables is a world of one); the process
    group (NCCL on GPUs, gloo on CPU) is used for rendezvous, for the baseline collectives and
    as the fallback when peer memory cannot be mapped.
  * `SymmetricBuffer` allocates device memory that every rank maps into its own address
    space (CUDA VMM handles exchanged by PyTorch's symmetric-memory rendezvous) and a signal
    pad per rank; the kernels that move data over NVLink are this package's own
    (csrc/comm/comm_kernels.cu) and take the per-rank address tables built here.
"""
from __future__ import annotations

import datetime
import os
from typing import Optional

import torch
import torch.distributed as dist

from .. import _backend as B

_state = {"initialized": False, "rank": 0, "world": 1, "local_rank": 0, "own_pg": False,
          "epoch": 0, "status": None}

SIGNAL_PAD_BYTES = 1024   # uint32 words: start [0,16), done [16,32), ticket 32, own epoch counter 33


def available() -> bool:
    return dist.is_available()


def num_gpus() -> int:
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def is_initialized() -> bool:
    return _state["initialized"]


def rank() -> int:
    return _state["rank"]


def world_size() -> int:
    return _state["world"]


def local_rank() -> int:
    return _state["local_rank"]


def init(num_gpus_: Optional[int] = None, backend: Optional[str] = None,
         timeout_s: float = 600.0) -> bool:
    """Join the job.  Returns True on success (the reference's init returns a boolean)."""
    if _state["initialized"]:
        return True
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rk = int(os.environ.get("RANK", "0"))
    lrk = int(os.environ.get("LOCAL_RANK", str(rk)))
    use_cuda = torch.cuda.is_available()
    if use_cuda:
        torch.cuda.set_device(lrk % max(1, torch.cuda.device_count()))
    if world > 1:
        if not dist.is_initialized():
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29500")
            be = backend or ("nccl" if use_cuda else "gloo")
            kwargs = {}
            if use_cuda and be == "nccl":
                kwargs["device_id"] = torch.device("cuda", torch.cuda.current_device())
            dist.init_process_group(be, rank=rk, world_size=world,
                                    timeout=datetime.timedelta(seconds=timeout_s), **kwargs)
            _state["own_pg"] = True
    _state.update(initialized=True, rank=rk, world=world, local_rank=lrk)
    return True


def destroy() -> None:
    if _state["own_pg"] and dist.is_initialized():
        try:
            dist.destroy_process_group()
        except Exception:
            pass
    _state.update(initialized=False, rank=0, world=1, local_rank=0, own_pg=False)


def next_epoch() -> int:
    """Host-side collective sequence number; identical on every rank as long as all ranks
    issue the same collectives in the same order.  Only the all-gather GEMM takes it: the
    other collectives pass epoch 0 and number themselves from a counter in their signal pad,
    which lets a captured CUDA graph be replayed."""
    _state["epoch"] += 1
    return _state["epoch"]


def barrier() -> None:
    if world_size() > 1:
        dist.barrier()


class SymmetricBuffer:
    """`nbytes` of device memory mapped on every rank, preceded by a signal pad.

    `ptrs` / `signal_ptrs` are int64 CUDA tensors with one address per rank (entry `rank` is
    the local one).  With a world of one (or when symmetric memory cannot be set up and
    `required` is False) the buffer is ordinary device memory and `peer_mapped` is False."""

    def __init__(self, nbytes: int, required: bool = False):
        self.nbytes = int(nbytes)
        self.peer_mapped = False
        self.multicast_ptr = 0
        total = SIGNAL_PAD_BYTES + (self.nbytes + 255) // 256 * 256
        dev = torch.device("cuda", torch.cuda.current_device())
        self.error: Optional[str] = None
        if world_size() > 1:
            try:
                import torch.distributed._symmetric_memory as symm_mem
                raw = symm_mem.empty(total, dtype=torch.uint8, device=dev)
                hdl = symm_mem.rendezvous(raw, dist.group.WORLD)
                self._hdl = hdl
                self.raw = raw
                bases = [int(p) for p in hdl.buffer_ptrs]
                self.peer_mapped = True
                # NVLink multicast address of the same memory (0 when the machine or the
                # allocation has none): what multimem.ld_reduce / multimem.st address
                try:
                    self.multicast_ptr = int(hdl.multicast_ptr or 0)
                except Exception:
                    self.multicast_ptr = 0
            except Exception as e:  # pragma: no cover - depends on the machine
                self.error = repr(e)
                if required:
                    raise
        if not self.peer_mapped:
            self.raw = torch.zeros(total, dtype=torch.uint8, device=dev)
            bases = [self.raw.data_ptr()] * world_size()
        self.raw.zero_()
        self.signal = self.raw[:SIGNAL_PAD_BYTES].view(torch.int32)
        self.data = self.raw[SIGNAL_PAD_BYTES:SIGNAL_PAD_BYTES + self.nbytes]
        self.signal_ptrs = torch.tensor(bases, dtype=torch.int64, device=dev)
        self.ptrs = torch.tensor([b + SIGNAL_PAD_BYTES for b in bases], dtype=torch.int64, device=dev)
        if world_size() > 1:
            torch.cuda.synchronize()
            dist.barrier()   # every rank's pad is zeroed before anyone signals

    def typed(self, dtype: torch.dtype) -> torch.Tensor:
        return self.data.view(dtype)


def status_buffer() -> torch.Tensor:
    if _state["status"] is None:
        _state["status"] = torch.zeros(8, dtype=torch.int32, device="cuda")
    return _state["status"]


class CommError(RuntimeError):
    """A device-side wait ran out of its budget; `.record` holds what the kernel saw."""

    def __init__(self, record):
        self.record = record
        super().__init__("luatorch_b200 collective failed: code=%d rank=%d epoch=%d phase=%d "
                         "peer=%d seen=%d" % tuple(record[:6]))


def check_status() -> None:
    """Raise CommError if any collective kernel recorded a timed-out wait (one device read)."""
    st = _state["status"]
    if st is None:
        return
    rec = st.tolist()
    if rec[0] != 0:
        st.zero_()
        raise CommError(rec)


# ------------------------------------------------------------------------------ collectives
def allreduce_mean_(t: torch.Tensor, buf: Optional[SymmetricBuffer] = None) -> torch.Tensor:
    """In-place average over ranks.  With a peer-mapped staging buffer the reduction is this
    package's two-shot peer-memory kernel; otherwise the process group's all_reduce."""
    w = world_size()
    if w == 1:
        return t
    if buf is not None and buf.peer_mapped and t.is_cuda and t.dtype in (torch.float32, torch.bfloat16):
        esz = t.element_size()
        vec = 16 // esz
        n = t.numel()
        pad = (-n) % (vec * w)
        if (n + pad) * esz <= buf.nbytes:
            stage = buf.typed(t.dtype)[:n + pad]
            stage[:n].copy_(t.reshape(-1))
            if pad:
                stage[n:].zero_()
            B.ext().peer_allreduce(buf.ptrs, buf.signal_ptrs, rank(), w, 0, n + pad,
                                   0 if t.dtype == torch.float32 else 1, 1.0 / w, 0,
                                   status_buffer())
            t.copy_(stage[:n].reshape(t.shape))
            return t
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    t.div_(w) if t.is_floating_point() else None
    return t


def broadcast_(t: torch.Tensor, root: int = 0, buf: Optional[SymmetricBuffer] = None) -> torch.Tensor:
    w = world_size()
    if w == 1:
        return t
    if buf is not None and buf.peer_mapped and t.is_cuda and t.numel() * t.element_size() <= buf.nbytes:
        nbytes = t.numel() * t.element_size()
        stage = buf.data[:nbytes]
        if rank() == root:
            stage.copy_(t.contiguous().view(torch.uint8).reshape(-1))
        B.ext().peer_broadcast(buf.ptrs, buf.signal_ptrs, rank(), w, root, 0, nbytes, 0,
                               status_buffer())
        if rank() != root:
            t.copy_(stage.view(t.dtype).reshape(t.shape))
        return t
    dist.broadcast(t, src=root)
    return t


# ------------------------------------------------------------------------------ all-gather + GEMM
class ShardedWeight:
    """A [K, N] bf16 weight whose row shards are owned by the ranks (rank p owns rows
    [p K/world, (p+1) K/world)): every rank holds a full-size copy in peer-mapped memory, of
    which only its own shard has to be current.  `gather_matmul` brings the other shards in
    from inside the GEMM kernel that consumes the weight.  (No counterpart in the reference,
    which has no sharding: lua/luatorch/distributed/ddp.lua.)"""

    def __init__(self, K: int, N: int):
        assert K % max(1, world_size()) == 0 and N % 8 == 0
        self.K, self.N = K, N
        self.buf = SymmetricBuffer(K * N * 2)
        self.weight = self.buf.typed(torch.bfloat16)[: K * N].view(K, N)
        self.flags = torch.zeros(world_size() + 1, dtype=torch.int32, device=self.weight.device)

    @property
    def shard(self) -> torch.Tensor:
        r, w = rank(), world_size()
        rows = self.K // w
        return self.weight[r * rows:(r + 1) * rows]


def gather_matmul(x: torch.Tensor, w: ShardedWeight, bias: Optional[torch.Tensor] = None,
                  gelu: bool = False, done_barrier: bool = True) -> torch.Tensor:
    """y = x @ W (+ bias, GELU) with the all-gather of W's row shards fused into the tcgen05
    GEMM: the kernel pulls the remote shards over NVLink into the local copy while its first
    tiles already multiply the local shard, so the transfer overlaps the math and each remote
    byte crosses the link once.  On return (stream order) `w.weight` is complete on this rank."""
    M, K = x.shape
    assert K == w.K and x.dtype == torch.bfloat16 and x.is_contiguous()
    y = torch.empty(M, w.N, dtype=torch.bfloat16, device=x.device)
    ws = world_size()
    if ws > 1 and w.buf.peer_mapped and M > 128:
        B.ext().gemm_gather(x, w.weight, y, M, w.N, K, K, w.N, w.N, bias, 1 if gelu else 0, None,
                            w.buf.ptrs, w.buf.signal_ptrs, w.flags, rank(), ws, next_epoch(),
                            status_buffer(), done_barrier)
        return y
    if ws > 1:   # unfused fallback: collective all-gather of the shards, then the plain GEMM
        parts = [torch.empty_like(w.shard) for _ in range(ws)]
        dist.all_gather(parts, w.shard.contiguous())
        w.weight.copy_(torch.cat(parts, 0))
    B.ext().gemm(x, w.weight, y, M, w.N, K, K, w.N, w.N, False, True, 1, 1, 0, 0, 0, 0, 0, 0, 1.0,
                 False, bias, 1 if gelu else 0, None, 0, None, None, 0, 0)
    return y
