"""Tensor front end.

Mirrors the `Tensor` class of the reference front end (lua/luatorch/tensor.lua:271-735):
`Tensor.new(shape, dtype, device)`, the fill / transfer / access methods, the static op
set (`Tensor.add`, `Tensor.matmul`, `Tensor.fused_layernorm`, ...) and the arithmetic
operators.  Storage is a `torch.Tensor`; on CUDA every op runs one of this package's own
sm_100a kernels through the `_C` extension, on CPU it runs the PyTorch CPU op with the
reference's edge-case behaviour (division by zero gives 0, sqrt of a negative gives 0,
log of a non-positive value gives -inf, shape errors return None after printing
`luatorch error: ...`).

Differences from the reference that are deliberate:
  * `reshape` exists (the reference calls it from nn/multihead.lua:66-68 but never defines it).
  * `bfloat16` is a first-class dtype (the reference has no reduced-precision compute).
  * `get`/`set` work on CUDA tensors (one element round trip) instead of printing an error.
  * a seedable RNG (`luatorch_b200.manual_seed`); the reference seeds from `time()`.
"""
from __future__ import annotations

import sys
from typing import List, Optional, Sequence

import torch

from . import _backend as B

_DTYPES = {
    "float32": torch.float32,
    "float64": torch.float64,
    "int32": torch.int32,
    "int64": torch.int64,
    "float16": torch.float16,
    "bfloat16": torch.bfloat16,
}
_DTYPE_NAMES = {v: k for k, v in _DTYPES.items()}


def _err(msg: str):
    print(f"luatorch error: {msg}", file=sys.stderr)
    return None


class Tensor:
    """Dense tensor with the reference's object surface (`shape`, `ndim`, `dtype`, `device`)."""

    __slots__ = ("_t", "requires_grad", "grad", "_node", "_grad_buf", "_compute", "_hook", "name",
                 "_unit", "_base", "_base_slice", "_act_ctx", "_bias_src")

    def __init__(self, shape=None, dtype: str = "float32", device: str = "cpu", _data=None):
        if _data is not None:
            self._t = _data
        else:
            if isinstance(shape, int):
                shape = [shape]
            self._t = torch.zeros(list(shape), dtype=_DTYPES[dtype],
                                  device="cuda" if device == "cuda" else "cpu")
        self.requires_grad = False
        self.grad = None
        self._node = None
        self._grad_buf = None     # preallocated gradient storage (parameter arenas)
        self._compute = None      # reduced-precision shadow used by kernels (bf16 copy of a master)
        self._hook = None         # called when the gradient of this tensor is final
        self.name = None
        self._unit = False        # True for the all-ones seed gradient of backward()
        self._base = None         # fused parameter this tensor is a column slice of
        self._base_slice = None
        self._act_ctx = None      # (activation, pre-activation) of a fused Linear output
        self._bias_src = None     # [bias parameter, done flag] of the Linear that produced this
                                  # tensor with a fused residual add (see nn/layernorm.py)

    # ------------------------------------------------------------------ construction
    @staticmethod
    def new(shape, dtype: str = "float32", device: str = "cpu") -> "Tensor":
        return Tensor(shape, dtype, device)

    @staticmethod
    def wrap(t: torch.Tensor) -> "Tensor":
        return Tensor(_data=t)

    @staticmethod
    def from_list(values, shape=None, dtype: str = "float32", device: str = "cpu") -> "Tensor":
        t = torch.tensor(values, dtype=_DTYPES[dtype])
        if shape is not None:
            t = t.reshape(list(shape))
        if device == "cuda":
            t = t.cuda()
        return Tensor(_data=t)

    # ------------------------------------------------------------------ properties
    @property
    def shape(self) -> List[int]:
        return list(self._t.shape)

    @property
    def ndim(self) -> int:
        return self._t.dim()

    @property
    def dtype(self) -> str:
        return _DTYPE_NAMES[self._t.dtype]

    @property
    def device(self) -> str:
        return "cuda" if self._t.is_cuda else "cpu"

    def numel(self) -> int:
        return self._t.numel()

    def torch(self) -> torch.Tensor:
        """The underlying storage (shared, not a copy)."""
        return self._t

    # ------------------------------------------------------------------ transfers
    def cuda(self) -> "Tensor":
        if not self._t.is_cuda:
            self._t = self._t.cuda()
        return self

    def cpu(self) -> "Tensor":
        if self._t.is_cuda:
            self._t = self._t.cpu()
        return self

    def cuda_async(self) -> "Tensor":
        """Host-to-device copy on the transfer stream from pinned memory; `Tensor.sync()`
        (or any later op, which waits on the copy's event) orders it before use."""
        if not self._t.is_cuda:
            self._t = B.async_to_cuda(self._t)
        return self

    def cpu_async(self) -> "Tensor":
        if self._t.is_cuda:
            self._t = B.async_to_cpu(self._t)
        return self

    @staticmethod
    def sync() -> None:
        B.sync_transfers()

    def to(self, dtype: str) -> "Tensor":
        """Cast to another dtype (new tensor)."""
        return Tensor(_data=B.cast(self._t, _DTYPES[dtype]))

    # ------------------------------------------------------------------ fills
    def fill(self, value: float) -> "Tensor":
        self._t.fill_(value)
        return self

    def zeros(self) -> "Tensor":
        self._t.zero_()
        return self

    def ones(self) -> "Tensor":
        self._t.fill_(1)
        return self

    def rand(self) -> "Tensor":
        B.fill_uniform(self._t)
        return self

    def randn(self) -> "Tensor":
        B.fill_normal(self._t)
        return self

    def print(self) -> "Tensor":
        flat = self._t.detach().float().reshape(-1)[:20].cpu().tolist()
        body = ", ".join(f"{v:.4f}" for v in flat)
        more = ", ..." if self.numel() > 20 else ""
        print(f"Tensor(shape=[{', '.join(str(s) for s in self.shape)}], data=[{body}{more}])")
        return self

    def copy(self) -> "Tensor":
        out = Tensor(_data=self._t.clone())
        out.requires_grad = self.requires_grad
        return out

    def copy_data(self, src: "Tensor") -> "Tensor":
        if src.numel() != self.numel():
            _err("copy_data size mismatch")
            return self
        self._t.copy_(src._t.reshape(self._t.shape))
        return self

    def get(self, idx: int) -> float:
        n = self.numel()
        if idx < 0 or idx >= n:
            _err(f"index {idx} out of bounds for tensor with {n} elements")
            return 0.0
        return float(self._t.reshape(-1)[idx].item())

    def set(self, idx: int, value: float) -> "Tensor":
        n = self.numel()
        if idx < 0 or idx >= n:
            _err(f"index {idx} out of bounds for tensor with {n} elements")
            return self
        if self._t.is_contiguous():
            self._t.view(-1)[idx] = value
        else:
            self._t[tuple(int(i) for i in torch.unravel_index(torch.tensor(idx), self._t.shape))] = value
        return self

    def reshape(self, shape: Sequence[int]) -> "Tensor":
        """View with a new shape sharing storage (csrc/tensor.c:260-294 in the reference)."""
        n = 1
        for s in shape:
            n *= s
        if n != self.numel():
            return _err("reshape size mismatch")
        return Tensor(_data=self._t.reshape(list(shape)))

    def item(self) -> float:
        return float(self._t.reshape(-1)[0].item())

    def tolist(self):
        return self._t.detach().float().cpu().tolist()

    def __repr__(self) -> str:
        return "Tensor(shape=%s, dtype=%s, device=%s)" % (
            "x".join(str(s) for s in self.shape), self.dtype, self.device)

    def __str__(self) -> str:
        return self.__repr__()

    # ------------------------------------------------------------------ operators
    def __add__(self, other):
        return Tensor.add(self, other) if isinstance(other, Tensor) else Tensor.add_scalar(self, other)

    def __sub__(self, other):
        return Tensor.sub(self, other) if isinstance(other, Tensor) else Tensor.add_scalar(self, -other)

    def __mul__(self, other):
        return Tensor.mul(self, other) if isinstance(other, Tensor) else Tensor.mul_scalar(self, other)

    def __truediv__(self, other):
        return Tensor.div(self, other) if isinstance(other, Tensor) else Tensor.div_scalar(self, other)

    def __neg__(self):
        return Tensor.neg(self)

    # ------------------------------------------------------------------ elementwise
    @staticmethod
    def _binary(name: str, a: "Tensor", b: "Tensor") -> Optional["Tensor"]:
        if a.numel() != b.numel():
            return _err(f"{name} size mismatch ({a.numel()} vs {b.numel()})")
        return Tensor(_data=B.binary(name, a._t, b._t))

    @staticmethod
    def add(a, b):
        return Tensor._binary("add", a, b)

    @staticmethod
    def sub(a, b):
        return Tensor._binary("sub", a, b)

    @staticmethod
    def mul(a, b):
        return Tensor._binary("mul", a, b)

    @staticmethod
    def div(a, b):
        return Tensor._binary("div", a, b)

    @staticmethod
    def add_scalar(a, s):
        return Tensor(_data=B.scalar_op("add", a._t, float(s)))

    @staticmethod
    def mul_scalar(a, s):
        return Tensor(_data=B.scalar_op("mul", a._t, float(s)))

    @staticmethod
    def div_scalar(a, s):
        if s == 0:
            _err("division by zero scalar")
            return Tensor(_data=torch.zeros_like(a._t))
        return Tensor(_data=B.scalar_op("div", a._t, float(s)))

    @staticmethod
    def pow_scalar(a, e):
        return Tensor(_data=B.scalar_op("pow", a._t, float(e)))

    @staticmethod
    def neg(a):
        return Tensor(_data=B.unary("neg", a._t))

    @staticmethod
    def abs(a):
        return Tensor(_data=B.unary("abs", a._t))

    @staticmethod
    def sqrt(a):
        return Tensor(_data=B.unary("sqrt", a._t))

    @staticmethod
    def log(a):
        return Tensor(_data=B.unary("log", a._t))

    @staticmethod
    def exp(a):
        return Tensor(_data=B.unary("exp", a._t))

    # ------------------------------------------------------------------ reductions
    @staticmethod
    def sum(a) -> float:
        return B.reduce("sum", a._t)

    @staticmethod
    def mean(a) -> float:
        return B.reduce("mean", a._t)

    @staticmethod
    def max(a) -> float:
        return B.reduce("max", a._t)

    @staticmethod
    def min(a) -> float:
        return B.reduce("min", a._t)

    # ------------------------------------------------------------------ in place
    @staticmethod
    def add_(a, b):
        if a.numel() != b.numel():
            _err("add_ size mismatch")
            return a
        B.binary_inplace("add", a._t, b._t)
        return a

    @staticmethod
    def sub_(a, b):
        if a.numel() != b.numel():
            _err("sub_ size mismatch")
            return a
        B.binary_inplace("sub", a._t, b._t)
        return a

    @staticmethod
    def mul_scalar_(a, s):
        B.scalar_inplace("mul", a._t, float(s))
        return a

    @staticmethod
    def add_scalar_(a, s):
        B.scalar_inplace("add", a._t, float(s))
        return a

    @staticmethod
    def add_broadcast(a, b):
        """[rows, cols] + [cols]."""
        if a.ndim != 2 or b.numel() != a.shape[1]:
            return _err("add_broadcast expects [rows, cols] + [cols]")
        return Tensor(_data=B.add_broadcast(a._t, b._t))

    @staticmethod
    def add_broadcast_backward(grad):
        """Column sum of a [rows, cols] gradient -> [cols]."""
        if grad.ndim != 2:
            return _err("add_broadcast_backward expects a 2-d tensor")
        return Tensor(_data=B.column_sum(grad._t))

    # ------------------------------------------------------------------ matmul family
    @staticmethod
    def matmul(a, b):
        if a.ndim != 2 or b.ndim != 2 or a.shape[1] != b.shape[0]:
            return _err(f"matmul shape mismatch {a.shape} x {b.shape}")
        return Tensor(_data=B.matmul(a._t, b._t))

    @staticmethod
    def bmm(a, b):
        if a.ndim != 3 or b.ndim != 3 or a.shape[0] != b.shape[0] or a.shape[2] != b.shape[1]:
            return _err(f"bmm shape mismatch {a.shape} x {b.shape}")
        return Tensor(_data=B.bmm(a._t, b._t))

    @staticmethod
    def transpose(a):
        if a.ndim != 2:
            return _err("transpose expects a 2-d tensor")
        return Tensor(_data=B.transpose(a._t))

    @staticmethod
    def dot(a, b) -> float:
        if a.numel() != b.numel():
            _err("dot size mismatch")
            return 0.0
        return B.dot(a._t, b._t)

    # ------------------------------------------------------------------ activations
    @staticmethod
    def relu(a):
        return Tensor(_data=B.unary("relu", a._t))

    @staticmethod
    def sigmoid(a):
        return Tensor(_data=B.unary("sigmoid", a._t))

    @staticmethod
    def tanh(a):
        return Tensor(_data=B.unary("tanh", a._t))

    @staticmethod
    def gelu(a):
        return Tensor(_data=B.unary("gelu", a._t))

    @staticmethod
    def silu(a):
        return Tensor(_data=B.unary("silu", a._t))

    @staticmethod
    def softmax(a):
        """Row softmax for 2-d input, whole-tensor softmax for 1-d."""
        return Tensor(_data=B.softmax(a._t))

    @staticmethod
    def gt_scalar(a, s):
        return Tensor(_data=B.scalar_op("gt", a._t, float(s)))

    # ------------------------------------------------------------------ losses
    @staticmethod
    def mse_loss(pred, target):
        if pred.numel() != target.numel():
            return _err("mse_loss size mismatch")
        return Tensor(_data=B.mse_loss(pred._t, target._t))

    @staticmethod
    def mse_loss_backward(pred, target):
        return Tensor(_data=B.mse_loss_backward(pred._t, target._t))

    @staticmethod
    def mae_loss(pred, target):
        if pred.numel() != target.numel():
            return _err("mae_loss size mismatch")
        return Tensor(_data=B.mae_loss(pred._t, target._t))

    @staticmethod
    def mae_loss_backward(pred, target):
        return Tensor(_data=B.mae_loss_backward(pred._t, target._t))

    @staticmethod
    def cross_entropy_loss(pred, target):
        """Mean cross entropy of raw logits [batch, classes] against float class labels."""
        if pred.ndim != 2 or target.numel() != pred.shape[0]:
            return _err("cross_entropy_loss expects logits [batch, classes] and labels [batch]")
        out = B.cross_entropy(pred._t, target._t)
        if out is None:
            return _err("cross_entropy_loss label out of range")
        return Tensor(_data=out)

    @staticmethod
    def cross_entropy_loss_backward(pred, target):
        return Tensor(_data=B.cross_entropy_backward(pred._t, target._t))

    # ------------------------------------------------------------------ fused ops
    @staticmethod
    def fused_gelu_bias(x, bias):
        """gelu(x + bias[col]) in one pass (both devices; the reference's CPU fallback is broken)."""
        return Tensor(_data=B.gelu_bias(x._t, bias._t))

    @staticmethod
    def fused_layernorm(x, gamma, beta, eps: float = 1e-5):
        """LayerNorm over the last dimension (both devices; the reference returns nil on CPU)."""
        return Tensor(_data=B.layernorm(x._t, gamma._t, beta._t, eps)[0])

    @staticmethod
    def fused_adam(param, grad, m, v, lr, beta1, beta2, eps, bc1, bc2, wd) -> bool:
        """In-place decoupled-weight-decay Adam step (csrc/cuda/ops/fused.cu:132-158 semantics)."""
        B.adam_step(param._t, grad._t, m._t, v._t, lr, beta1, beta2, eps, bc1, bc2, wd)
        return True

    @staticmethod
    def flash_attention(Q, K, V, batch_heads, seq_len, head_dim, causal=True):
        """softmax(Q K^T / sqrt(d)) V over [batch_heads, seq, head_dim] inputs."""
        q = Q._t.reshape(batch_heads, seq_len, head_dim)
        k = K._t.reshape(batch_heads, seq_len, head_dim)
        v = V._t.reshape(batch_heads, seq_len, head_dim)
        return Tensor(_data=B.attention(q, k, v, bool(causal))[0])

    @staticmethod
    def has_inf_nan(t) -> bool:
        return B.has_inf_nan(t._t)

    @staticmethod
    def scale_(t, s):
        B.scalar_inplace("mul", t._t, float(s))
        return t

    @staticmethod
    def im2col(input, batch, channels, height, width, kernel_size, stride=1, padding=0):
        return Tensor(_data=B.im2col(input._t, batch, channels, height, width, kernel_size,
                                     stride, padding))

    # ------------------------------------------------------------------ memory pool
    @staticmethod
    def pool_init():
        B.pool_init()

    @staticmethod
    def pool_clear():
        B.pool_clear()

    @staticmethod
    def cuda_memory_allocated() -> int:
        return B.memory_allocated()

    @staticmethod
    def cuda_memory_cached() -> int:
        return B.memory_cached()
