"""`lf.distributed`: DDP, nccl, num_gpus, init, destroy (lua/luatorch/init.lua:49-61),
plus rank / world_size queries, peer-mapped memory and failure detection."""
from . import comm, elastic, nccl
from .comm import (CommError, ShardedWeight, SymmetricBuffer, available, barrier, check_status, destroy, init,
                   gather_matmul, is_initialized, local_rank, num_gpus, rank, world_size)
from .ddp import DDP
from .elastic import Heartbeat, RankFailure, StepFailed, resume, run_step_guarded

__all__ = ["DDP", "nccl", "comm", "elastic", "num_gpus", "init", "destroy", "rank", "world_size",
           "local_rank", "available", "barrier", "is_initialized", "SymmetricBuffer", "CommError",
           "check_status", "ShardedWeight", "gather_matmul", "Heartbeat", "RankFailure", "StepFailed", "resume", "run_step_guarded"]
