"""luatorch_b200: a Blackwell (B200, sm_100a) deep-learning framework with the capabilities
and public surface of luatorch.

The namespace mirrors the reference's `require('luatorch')` table
(lua/luatorch/init.lua:4-79):

    lf.Tensor, lf.autograd, lf.nn,
    lf.optim.{Adam, AdamW, SGD, CosineAnnealing, WarmupScheduler, StepLR},
    lf.data.{DataLoader, Tokenizer, TextDataset}, lf.models.{GPT, MLP},
    lf.io.checkpoint, lf.utils.{Logger, Config}, lf.cuda.amp,
    lf.distributed.{DDP, nccl, num_gpus, init, destroy}, lf.export.onnx, lf.version

PyTorch tensors are the storage layer; every CUDA op is one of this package's own sm_100a
kernels (tcgen05 / TMEM / TMA GEMM and flash attention, fused LayerNorm / GELU / softmax-CE /
embedding / optimizer kernels, peer-memory collectives fused with AdamW).
"""
import os as _os

version = "0.1.0"
__version__ = version

from . import _backend  # noqa: E402
from ._backend import manual_seed  # noqa: E402
from .tensor import Tensor  # noqa: E402
from . import autograd  # noqa: E402
from . import nn  # noqa: E402
from . import optim  # noqa: E402
from . import data  # noqa: E402
from . import models  # noqa: E402
from . import io  # noqa: E402
from . import utils  # noqa: E402
from . import parallel  # noqa: E402
from . import cuda  # noqa: E402
from . import distributed  # noqa: E402
from . import export  # noqa: E402
from . import ops  # noqa: E402


def launch_counts():
    """(gemm, memory-bound, attention, communication) kernel launches since import."""
    return _backend.launch_counts()


if _os.environ.get("LUAFLOW_DEBUG") or _os.environ.get("LUATORCH_DEBUG"):
    print("luatorch_b200 v%s" % version)
    print("  gpus: %d" % distributed.num_gpus())

__all__ = ["Tensor", "autograd", "nn", "optim", "data", "models", "io", "utils", "cuda",
           "distributed", "export", "parallel", "ops", "manual_seed", "version", "launch_counts"]
