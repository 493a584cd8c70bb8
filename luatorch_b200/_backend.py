"""Device dispatch for tensor ops.

CUDA tensors go to this package's own sm_100a kernels (`luatorch_b200._C`); CPU tensors use
PyTorch's CPU ops with the reference's edge-case behaviour (csrc/ops/arithmetic.c:61-65,
132-152).  There is no silent fallback: a CUDA tensor without the compiled extension raises.

The reference does this dispatch in Lua on the device of the first operand only
(lua/luatorch/tensor.lua:437-646).
"""
from __future__ import annotations

import math
import threading
from typing import Optional, Tuple

import torch

from .utils import debug as _debug

_C = None
_C_error: Optional[BaseException] = None


def _load_ext():
    global _C, _C_error
    if _C is not None or _C_error is not None:
        return _C
    try:
        from . import _C as ext  # type: ignore
        _C = ext
    except Exception as e:  # built lazily on first use if the shared object is missing
        try:
            from .build import build_all
            build_all(abi=False)
            from . import _C as ext  # type: ignore
            _C = ext
        except Exception as e2:
            _C_error = e2
            _C = None
    return _C


def ext():
    """The compiled kernel module; raises if it cannot be loaded."""
    c = _load_ext()
    if c is None:
        raise RuntimeError(
            "luatorch_b200: the sm_100a kernel extension (_C) is not available: %r. "
            "Run `python -m luatorch_b200.build`." % (_C_error,))
    return c


_BIN = {"add": 0, "sub": 1, "mul": 2, "div": 3}
_SC = {"add": 0, "mul": 1, "div": 2, "pow": 3, "gt": 4}
_UN = {"neg": 0, "abs": 1, "sqrt": 2, "log": 3, "exp": 4, "relu": 5, "sigmoid": 6, "tanh": 7,
       "gelu": 8, "silu": 9}
_KERNEL_DTYPES = (torch.float32, torch.bfloat16, torch.float16)

# ------------------------------------------------------------------------------ RNG
_rng_lock = threading.Lock()
_seed = 0x5EED
_offset = 0
_cpu_gen = torch.Generator(device="cpu")
_cpu_gen.manual_seed(_seed)


def manual_seed(seed: int) -> None:
    """Seed both the CPU generator and the Philox stream used by the CUDA kernels."""
    global _seed, _offset
    with _rng_lock:
        _seed = int(seed)
        _offset = 0
        _cpu_gen.manual_seed(_seed)


def next_philox(n_elements: int) -> Tuple[int, int]:
    """Reserve a slice of the Philox counter space; returns (seed, offset)."""
    global _offset
    with _rng_lock:
        off = _offset
        _offset += (int(n_elements) + 3) // 4 + 1
        return _seed, off


def rng_state() -> dict:
    return {"seed": _seed, "offset": _offset, "cpu": _cpu_gen.get_state()}


def set_rng_state(state: dict) -> None:
    global _seed, _offset
    with _rng_lock:
        _seed, _offset = int(state["seed"]), int(state["offset"])
        _cpu_gen.set_state(state["cpu"])


def cpu_generator() -> torch.Generator:
    return _cpu_gen


def fill_uniform(t: torch.Tensor) -> None:
    if t.is_cuda:
        seed, off = next_philox(t.numel())
        if t.dtype in _KERNEL_DTYPES and t.is_contiguous():
            ext().fill_random(t, seed, off, False)
        else:
            tmp = torch.empty(t.shape, device=t.device, dtype=torch.float32)
            ext().fill_random(tmp, seed, off, False)
            t.copy_(tmp)
    else:
        t.copy_(torch.rand(t.shape, generator=_cpu_gen).to(t.dtype))


def fill_normal(t: torch.Tensor) -> None:
    if t.is_cuda:
        seed, off = next_philox(t.numel())
        if t.dtype in _KERNEL_DTYPES and t.is_contiguous():
            ext().fill_random(t, seed, off, True)
        else:
            tmp = torch.empty(t.shape, device=t.device, dtype=torch.float32)
            ext().fill_random(tmp, seed, off, True)
            t.copy_(tmp)
    else:
        t.copy_(torch.randn(t.shape, generator=_cpu_gen).to(t.dtype))


# ------------------------------------------------------------------------------ transfers
_xfer_stream = None
_xfer_events = []


def _transfer_stream():
    global _xfer_stream
    if _xfer_stream is None:
        _xfer_stream = torch.cuda.Stream()
    return _xfer_stream


def async_to_cuda(t: torch.Tensor) -> torch.Tensor:
    """Pinned staging + copy on the transfer stream; the compute stream waits on the copy's
    event, so later ops are ordered after it without a host synchronise (the reference's
    "async" copies use pageable memory and therefore never overlap,
    csrc/cuda/tensor.cu:126-181)."""
    src = t if t.is_pinned() else t.contiguous().pin_memory()
    s = _transfer_stream()
    with torch.cuda.stream(s):
        out = src.to("cuda", non_blocking=True)
    ev = torch.cuda.Event()
    ev.record(s)
    torch.cuda.current_stream().wait_event(ev)
    out.record_stream(torch.cuda.current_stream())
    _xfer_events.append((ev, src))
    if len(_xfer_events) > 64:
        _xfer_events[:] = [(e, h) for (e, h) in _xfer_events if not e.query()]
    return out


def async_to_cpu(t: torch.Tensor) -> torch.Tensor:
    s = _transfer_stream()
    s.wait_stream(torch.cuda.current_stream())
    out = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
    with torch.cuda.stream(s):
        out.copy_(t, non_blocking=True)
    t.record_stream(s)
    ev = torch.cuda.Event()
    ev.record(s)
    _xfer_events.append((ev, out))
    return out


def sync_transfers() -> None:
    if _xfer_stream is not None:
        _xfer_stream.synchronize()
    _xfer_events.clear()


# ------------------------------------------------------------------------------ helpers
def _k(t: torch.Tensor) -> torch.Tensor:
    """Kernel-ready view of a CUDA tensor (contiguous, kernel dtype)."""
    if t.dtype not in _KERNEL_DTYPES:
        t = t.float()
    return t if t.is_contiguous() else t.contiguous()


def cast(t: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    if t.dtype == dtype:
        return t.clone()
    if t.is_cuda and t.dtype in _KERNEL_DTYPES and dtype in _KERNEL_DTYPES:
        return ext().cast(_k(t), dtype)
    return t.to(dtype)


# ------------------------------------------------------------------------------ elementwise
def binary(name: str, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    if a.is_cuda:
        b = b if b.dtype == a.dtype else b.to(a.dtype)
        return ext().binary(_BIN[name], _k(a), _k(b).reshape(a.shape), False)
    b = b.reshape(a.shape)
    if name == "add":
        return a + b
    if name == "sub":
        return a - b
    if name == "mul":
        return a * b
    out = a / b
    return torch.where(b == 0, torch.zeros_like(out), out)  # x / 0 -> 0 like the C op


def binary_inplace(name: str, a: torch.Tensor, b: torch.Tensor) -> None:
    if a.is_cuda and a.is_contiguous() and a.dtype in _KERNEL_DTYPES:
        b = b if b.dtype == a.dtype else b.to(a.dtype)
        ext().binary(_BIN[name], a, _k(b).reshape(a.shape), True)
        return
    if name == "add":
        a.add_(b.reshape(a.shape))
    else:
        a.sub_(b.reshape(a.shape))


def scalar_op(name: str, a: torch.Tensor, s: float) -> torch.Tensor:
    if a.is_cuda:
        return ext().scalar(_SC[name], _k(a), s, False)
    if name == "add":
        return a + s
    if name == "mul":
        return a * s
    if name == "div":
        return a / s
    if name == "pow":
        return torch.pow(a, s)
    return (a > s).to(a.dtype)


def scalar_inplace(name: str, a: torch.Tensor, s: float) -> None:
    if a.is_cuda and a.is_contiguous() and a.dtype in _KERNEL_DTYPES:
        ext().scalar(_SC[name], a, s, True)
        return
    if name == "add":
        a.add_(s)
    else:
        a.mul_(s)


def _gelu_cpu(x):
    return 0.5 * x * (1.0 + torch.tanh(0.7978845608 * (x + 0.044715 * x * x * x)))


def unary(name: str, a: torch.Tensor) -> torch.Tensor:
    if a.is_cuda:
        return ext().unary(_UN[name], _k(a))
    if name == "neg":
        return -a
    if name == "abs":
        return a.abs()
    if name == "sqrt":
        return torch.where(a < 0, torch.zeros_like(a), a.clamp_min(0).sqrt())
    if name == "log":
        return torch.where(a <= 0, torch.full_like(a, -math.inf), a.clamp_min(1e-45).log())
    if name == "exp":
        return a.exp()
    if name == "relu":
        return a.clamp_min(0)
    if name == "sigmoid":
        return torch.sigmoid(a)
    if name == "tanh":
        return torch.tanh(a)
    if name == "gelu":
        return _gelu_cpu(a)
    if name == "silu":
        return a * torch.sigmoid(a)
    raise ValueError(name)


def unary_backward(name: str, x: torch.Tensor, dy: torch.Tensor) -> torch.Tensor:
    """dy * f'(x)."""
    if x.is_cuda:
        return ext().unary_backward(_UN[name], _k(x), _k(dy.to(x.dtype)).reshape(x.shape))
    dy = dy.reshape(x.shape)
    if name == "relu":
        return dy * (x > 0).to(x.dtype)
    if name == "sigmoid":
        s = torch.sigmoid(x)
        return dy * s * (1 - s)
    if name == "tanh":
        t = torch.tanh(x)
        return dy * (1 - t * t)
    if name == "gelu":
        k0, k1 = 0.7978845608, 0.044715
        t = torch.tanh(k0 * (x + k1 * x ** 3))
        return dy * (0.5 * (1 + t) + 0.5 * x * (1 - t * t) * k0 * (1 + 3 * k1 * x * x))
    if name == "silu":
        s = torch.sigmoid(x)
        return dy * (s + x * s * (1 - s))
    raise ValueError(name)


def reduce(name: str, a: torch.Tensor) -> float:
    if a.is_cuda:
        n = a.numel()
        if name == "sum":
            return float(ext().reduce(0, _k(a), 1.0).item())
        if name == "mean":
            return float(ext().reduce(0, _k(a), 1.0 / n).item())
        return float(ext().reduce(1 if name == "max" else 2, _k(a), 1.0).item())
    a = a.float()
    return float(getattr(a, name)().item())


def add_broadcast(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    if a.is_cuda:
        return ext().add_broadcast(_k(a), _k(b.to(a.dtype)).reshape(-1))
    return a + b.reshape(1, -1)


def column_sum(g: torch.Tensor, out: Optional[torch.Tensor] = None, accumulate: bool = False) -> torch.Tensor:
    if g.is_cuda:
        g = g if g.stride(-1) == 1 else g.contiguous()
        return ext().column_sum(g, out, accumulate)
    s = g.sum(0)
    if out is None:
        return s
    if accumulate:
        out.add_(s.to(out.dtype))
    else:
        out.copy_(s)
    return out


# Set by luatorch_b200.cuda.graph.GraphedStep while it captures a training step: an object with
# device tensors `dyn_opt` (fp32 {lr, bc1, bc2}) and `dyn_off` (int64 Philox offset).  Ops whose
# launch arguments change from step to step read them from there instead, so that the captured
# graph stays valid when it is replayed.
_graph_capture = None


def dropout(x: torch.Tensor, p: float) -> Tuple[torch.Tensor, object]:
    """Returns (y, ctx); ctx regenerates the same mask in `dropout_backward`."""
    if x.is_cuda:
        seed, off = next_philox(x.numel())
        cap = _graph_capture
        if cap is not None:
            return ext().dropout_dyn(_k(x), p, seed, off, cap.dyn_off), (seed, off, cap.dyn_off)
        return ext().dropout(_k(x), p, seed, off), (seed, off)
    mask = (torch.rand(x.shape, generator=_cpu_gen) >= p).to(x.dtype) / (1.0 - p if p < 1 else 1.0)
    return x * mask, mask


def dropout_backward(dy: torch.Tensor, p: float, ctx) -> torch.Tensor:
    if dy.is_cuda:
        if len(ctx) == 3:
            return ext().dropout_dyn(_k(dy), p, ctx[0], ctx[1], ctx[2])
        seed, off = ctx
        return ext().dropout(_k(dy), p, seed, off)
    return dy * ctx


# ------------------------------------------------------------------------------ matmul family
def gemm(a, b, *, a_t=False, b_t=False, out=None, out_dtype=None, alpha=1.0, accumulate=False,
         bias=None, act=0, residual=None, aux_out=None, aux_in=None, n_valid=None, k_valid=None,
         overlap_prev=0):
    """C = act(alpha * op(a) @ op(b) + bias) + residual on the tensor cores (bf16 operands).

    a: [M, K] (or [K, M] when a_t), b: [K, N] (or [N, K] when b_t); both 2-d with unit inner
    stride (row strides may exceed the logical width).  `n_valid` restricts the logical N when
    b is a padded buffer.  `overlap_prev=n`: the caller guarantees that this product reads
    nothing the n kernels launched just before it write and writes nothing they touch (`out`
    given, not freshly allocated); it then runs in their tail instead of after them.
    """
    C = ext()
    if a_t:
        K, M = a.shape
    else:
        M, K = a.shape
    if b_t:
        N = b.shape[0]
    else:
        N = b.shape[1]
    if n_valid is not None:
        N = n_valid
    if k_valid is not None:
        K = k_valid
    if out is None:
        out = torch.empty((M, N), device=a.device, dtype=out_dtype or torch.bfloat16)
    elif overlap_prev:
        C.gemm_next_overlaps_prev(int(overlap_prev))
    C.gemm(a, b, out, M, N, K, a.stride(0), b.stride(0), out.stride(0), bool(a_t), not b_t,
           1, 1, 0, 0, 0, 0, 0, 0, float(alpha), bool(accumulate), bias, int(act), residual,
           residual.stride(0) if residual is not None else 0, aux_out, aux_in,
           aux_in.stride(0) if aux_in is not None else 0, 0)
    if _debug._on:
        _debug.check_kernels(C)
    return out


def _matmul_fp32_tc(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """fp32-accurate product on bf16 tensor cores: a = a_hi + a_lo, b = b_hi + b_lo and
    a @ b ~= a_hi b_hi + a_hi b_lo + a_lo b_hi, evaluated as ONE GEMM over a 3x longer K."""
    C = ext()
    a_hi, a_lo = C.split_bf16(a)
    b_hi, b_lo = C.split_bf16(b)
    a3 = torch.cat([a_hi, a_hi, a_lo], dim=1)
    b3 = torch.cat([b_hi, b_lo, b_hi], dim=0)
    return gemm(a3, b3, out_dtype=torch.float32)


def matmul(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    if a.is_cuda:
        if a.dtype == torch.bfloat16:
            return gemm(_k(a), _k(b.to(torch.bfloat16)))
        return _matmul_fp32_tc(_k(a.float()), _k(b.float())).to(a.dtype)
    return a @ b


def bmm(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    if a.is_cuda:
        nb, M, K = a.shape
        N = b.shape[2]
        if a.dtype == torch.bfloat16:
            a_, b_ = _k(a), _k(b.to(torch.bfloat16))
            out = torch.empty((nb, M, N), device=a.device, dtype=torch.bfloat16)
        else:
            C = ext()
            a_hi, a_lo = C.split_bf16(_k(a.float()))
            b_hi, b_lo = C.split_bf16(_k(b.float()))
            a_ = torch.cat([a_hi, a_hi, a_lo], dim=2)
            b_ = torch.cat([b_hi, b_lo, b_hi], dim=1)
            K = 3 * K
            out = torch.empty((nb, M, N), device=a.device, dtype=torch.float32)
        ext().gemm(a_, b_, out, M, N, K, K, N, N, False, True, nb, 1, M * K, 0, K * N, 0, M * N, 0,
                   1.0, False, None, 0, None, 0, None, None, 0, 0)
        return out.to(a.dtype)
    return torch.bmm(a, b)


def transpose(a: torch.Tensor) -> torch.Tensor:
    if a.is_cuda:
        return ext().transpose2d(_k(a))
    return a.t().contiguous()


def dot(a: torch.Tensor, b: torch.Tensor) -> float:
    if a.is_cuda:
        return float(ext().dot(_k(a).reshape(-1), _k(b.to(a.dtype)).reshape(-1)).item())
    return float(torch.dot(a.reshape(-1).float(), b.reshape(-1).float()).item())


# ------------------------------------------------------------------------------ softmax / losses
def softmax(a: torch.Tensor) -> torch.Tensor:
    if a.is_cuda:
        return ext().softmax(_k(a))
    return torch.softmax(a, dim=-1) if a.dim() >= 2 else torch.softmax(a, dim=0)


def mse_loss(p, t):
    if p.is_cuda:
        return ext().pointwise_loss(0, _k(p), _k(t.to(p.dtype)).reshape(p.shape))
    return ((p - t.reshape(p.shape)) ** 2).mean().reshape(1)


def mse_loss_backward(p, t, scale: float = 1.0):
    if p.is_cuda:
        return ext().pointwise_loss_backward(0, _k(p), _k(t.to(p.dtype)).reshape(p.shape), scale)
    return 2.0 * (p - t.reshape(p.shape)) / p.numel() * scale


def mae_loss(p, t):
    if p.is_cuda:
        return ext().pointwise_loss(1, _k(p), _k(t.to(p.dtype)).reshape(p.shape))
    return (p - t.reshape(p.shape)).abs().mean().reshape(1)


def mae_loss_backward(p, t, scale: float = 1.0):
    if p.is_cuda:
        return ext().pointwise_loss_backward(1, _k(p), _k(t.to(p.dtype)).reshape(p.shape), scale)
    return torch.sign(p - t.reshape(p.shape)) / p.numel() * scale


def _labels(t: torch.Tensor) -> torch.Tensor:
    t = t.reshape(-1)
    if t.dtype in (torch.int64, torch.int32, torch.float32):
        return t.contiguous()
    return t.float().contiguous() if t.is_floating_point() else t.long().contiguous()


def cross_entropy_full(logits: torch.Tensor, labels: torch.Tensor, n_classes: Optional[int] = None):
    """Returns (loss[1] fp32, lse[rows] fp32) or None when a label is out of range.
    On CUDA the out-of-range check costs one device-to-host read of a flag; callers on the hot
    path use `cross_entropy_device` instead."""
    cols = n_classes or logits.shape[1]
    if logits.is_cuda:
        lg = logits if logits.stride(-1) == 1 else logits.contiguous()
        loss, lse, err = ext().cross_entropy_forward(lg, cols, _labels(labels))
        if int(err[0].item()) != 0:
            return None
        return loss, lse
    lab = labels.reshape(-1).long()
    if lab.numel() and (int(lab.min()) < 0 or int(lab.max()) >= cols):
        return None
    lg = logits[:, :cols].float()
    lse = torch.logsumexp(lg, dim=1)
    loss = (lse - lg.gather(1, lab.reshape(-1, 1)).reshape(-1)).mean().reshape(1)
    return loss, lse


def cross_entropy(logits, labels):
    r = cross_entropy_full(logits, labels)
    return None if r is None else r[0].to(torch.float32)


def cross_entropy_device(logits, labels, n_classes):
    """CUDA only, no host synchronisation: (loss, lse, err_flag) all on the device."""
    lg = logits if logits.stride(-1) == 1 else logits.contiguous()
    return ext().cross_entropy_forward(lg, n_classes, _labels(labels))


def cross_entropy_backward(logits, labels, lse=None, scale: float = 1.0, out=None,
                           n_classes: Optional[int] = None, scale_dev=None):
    cols = n_classes or logits.shape[1]
    rows = logits.shape[0]
    if logits.is_cuda:
        lg = logits if logits.stride(-1) == 1 else logits.contiguous()
        if lse is None:
            _, lse, _ = ext().cross_entropy_forward(lg, cols, _labels(labels))
        if out is None:
            out = torch.empty_like(lg)
        ext().cross_entropy_backward(lg, cols, _labels(labels), lse, scale / rows, scale_dev,
                                     out)
        return out
    lg = logits[:, :cols].float()
    p = torch.softmax(lg, dim=1)
    p[torch.arange(rows), labels.reshape(-1).long()] -= 1.0
    g = (p * (scale / rows)).to(logits.dtype)
    if out is not None:
        out[:, :cols].copy_(g)
        return out
    return g


# ------------------------------------------------------------------------------ fused ops
def gelu_bias(x, bias):
    if x.is_cuda:
        return ext().gelu_bias_forward(_k(x), None if bias is None else _k(bias))
    return _gelu_cpu(x + bias.reshape(1, -1).to(x.dtype))


def gelu_bias_backward(x, bias, dy):
    if x.is_cuda:
        return ext().gelu_bias_backward(_k(x), None if bias is None else _k(bias), _k(dy))
    z = x + (bias.reshape(1, -1).to(x.dtype) if bias is not None else 0)
    return unary_backward("gelu", z, dy)


def layernorm(x, gamma, beta, eps: float = 1e-5):
    """Returns (y, mean, rstd) over the last dimension."""
    if x.is_cuda:
        y, mean, rstd = ext().layernorm_forward(_k(x), _k(gamma), _k(beta), eps)
        return y, mean, rstd
    xf = x.float()
    mean = xf.mean(-1, keepdim=True)
    var = xf.var(-1, unbiased=False, keepdim=True)
    rstd = torch.rsqrt(var + eps)
    y = (xf - mean) * rstd * gamma.float() + beta.float()
    return y.to(x.dtype), mean.reshape(-1), rstd.reshape(-1)


def layernorm_backward(x, dy, gamma, mean, rstd, dgamma, dbeta, accumulate=False, dx_add=None):
    """Returns dx; writes (or accumulates) dgamma / dbeta."""
    if x.is_cuda:
        return ext().layernorm_backward(_k(x), _k(dy), _k(gamma), mean, rstd,
                                        None if dx_add is None else _k(dx_add), dgamma, dbeta,
                                        accumulate)
    cols = x.shape[-1]
    xf, dyf = x.float().reshape(-1, cols), dy.float().reshape(-1, cols)
    xh = (xf - mean.reshape(-1, 1)) * rstd.reshape(-1, 1)
    g = dyf * gamma.float()
    c1 = g.mean(-1, keepdim=True)
    c2 = (g * xh).mean(-1, keepdim=True)
    dx = rstd.reshape(-1, 1) * (g - c1 - xh * c2)
    if dx_add is not None:
        dx = dx + dx_add.float().reshape(-1, cols)
    dg, db = (dyf * xh).sum(0), dyf.sum(0)
    if accumulate:
        dgamma.add_(dg.to(dgamma.dtype))
        dbeta.add_(db.to(dbeta.dtype))
    else:
        dgamma.copy_(dg)
        dbeta.copy_(db)
    return dx.reshape(x.shape).to(x.dtype)


def adamw_flat(master, shadow, grad, m, v, seg_end, seg_wd, lr, beta1, beta2, eps, bc1, bc2,
               grad_scale, skip_flag) -> None:
    """One launch over a flat arena (csrc/kernels/optim.cu).  Under graph capture lr and the
    bias corrections are read from device memory."""
    cap = _graph_capture
    if cap is not None:
        cap.uses_optimizer = True
        ext().adamw_flat_dyn(master, shadow, grad, m, v, seg_end, seg_wd, lr, beta1, beta2, eps,
                             bc1, bc2, grad_scale, skip_flag, cap.dyn_opt)
    else:
        ext().adamw_flat(master, shadow, grad, m, v, seg_end, seg_wd, lr, beta1, beta2, eps, bc1,
                         bc2, grad_scale, skip_flag)


def sgd_flat(master, shadow, grad, vel, lr, momentum, nesterov, grad_scale) -> None:
    cap = _graph_capture
    if cap is not None:
        cap.uses_optimizer = True
        ext().sgd_flat_dyn(master, shadow, grad, vel, lr, momentum, nesterov, grad_scale,
                           cap.dyn_opt)
    else:
        ext().sgd_flat(master, shadow, grad, vel, lr, momentum, nesterov, grad_scale)


def adam_step(p, g, m, v, lr, beta1, beta2, eps, bc1, bc2, wd):
    if p.is_cuda:
        if _graph_capture is not None:
            raise RuntimeError("graph capture needs the parameters in a flat arena "
                               "(wrap the model in distributed.DDP before building the optimizer)")
        n = p.numel()
        ext().adamw_flat(p.view(-1), None, _k(g).view(-1), m.view(-1), v.view(-1),
                         torch.tensor([n], device=p.device, dtype=torch.int64),
                         torch.tensor([wd], device=p.device, dtype=torch.float32),
                         lr, beta1, beta2, eps, bc1, bc2, 1.0, None)
        return
    if wd:
        p.mul_(1.0 - lr * wd)
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    p.sub_(lr * (m / bc1) / ((v / bc2).sqrt() + eps))


def attention(q, k, v, causal: bool, scale: Optional[float] = None):
    """q, k, v: [BH, S, D]. Returns (o [BH, S, D], lse [BH, S])."""
    D = q.shape[-1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if q.is_cuda and D in (64, 128):
        dt = q.dtype
        q4, k4, v4 = (t.to(torch.bfloat16).contiguous().unsqueeze(2) for t in (q, k, v))  # [BH,S,1,D]
        o, lse = ext().flash_forward(q4, k4, v4, causal, scale)
        return o.squeeze(2).to(dt), lse.squeeze(1)
    if q.is_cuda and D % 8 == 0 and q.shape[1] % 8 == 0:
        # other head dims: scores, softmax and P V as batched tcgen05 GEMMs + the score-softmax
        # kernel (no library GEMM on the GPU); the log-sum-exp comes from the row maxima of P
        dt = q.dtype
        q4, k4, v4 = (t.to(torch.bfloat16).contiguous().unsqueeze(2) for t in (q, k, v))
        o, p = _attn_composed_forward(q4, k4, v4, causal, scale)
        # p holds softmax(s), so lse_i = s_ij - log p_ij for any key j: take each row's
        # largest probability (never rounded to zero) and recompute that one score in fp32
        pm, jm = p[:, 0].float().max(-1)                                   # [BH, S]
        kj = torch.gather(k4[:, :, 0].float(), 1, jm.unsqueeze(-1).expand(-1, -1, D))
        lse = (q4[:, :, 0].float() * kj).sum(-1) * scale - torch.log(pm)
        return o.squeeze(2).to(dt), lse
    qf, kf, vf = q.float(), k.float(), v.float()
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        S = q.shape[1]
        s = s.masked_fill(torch.triu(torch.ones(S, S, dtype=torch.bool, device=q.device), 1), -math.inf)
    lse = torch.logsumexp(s, -1)
    return torch.matmul(torch.softmax(s, -1), vf).to(q.dtype), lse


def has_inf_nan(t: torch.Tensor) -> bool:
    if t.is_cuda and t.dtype in _KERNEL_DTYPES and t.is_contiguous():
        flag = torch.zeros(1, device=t.device, dtype=torch.int32)
        ext().check_finite_scale(t, 1.0, False, flag)
        return bool(flag.item())
    return not bool(torch.isfinite(t).all().item())


def im2col(x, batch, C, H, W, k, stride, pad):
    if x.is_cuda:
        return ext().im2col(_k(x).reshape(-1), batch, C, H, W, k, stride, pad, 0)
    xx = x.reshape(batch, C, H, W).float()
    unf = torch.nn.functional.unfold(xx, k, padding=pad, stride=stride)
    return unf.transpose(1, 2).reshape(-1, C * k * k).contiguous().to(x.dtype)


def col2im(cols, batch, C, H, W, k, stride, pad):
    if cols.is_cuda:
        return ext().col2im(cols if cols.stride(-1) == 1 else cols.contiguous(), batch, C, H, W, k,
                            stride, pad)
    L = cols.shape[0] // batch
    g = cols.float().reshape(batch, L, -1).transpose(1, 2)
    return torch.nn.functional.fold(g, (H, W), k, padding=pad, stride=stride).reshape(-1).to(cols.dtype)


def relayout(x, batch, C, hw, to_nchw: bool):
    """[batch*hw, C] (NHWC-flat) <-> [batch, C, hw] (NCHW-flat), flat storage either way."""
    if x.is_cuda:
        return ext().relayout(_k(x).reshape(-1), batch, C, hw, to_nchw)
    if to_nchw:
        return x.reshape(batch, hw, C).transpose(1, 2).contiguous().reshape(-1)
    return x.reshape(batch, C, hw).transpose(1, 2).contiguous().reshape(-1)


# ------------------------------------------------------------------------------ memory pool
def pool_init():
    if torch.cuda.is_available():
        torch.cuda.init()


def pool_clear():
    if torch.cuda.is_available():
        torch.cuda.empty_cache()


def memory_allocated() -> int:
    return torch.cuda.memory_reserved() if torch.cuda.is_available() else 0


def memory_cached() -> int:
    if not torch.cuda.is_available():
        return 0
    return torch.cuda.memory_reserved() - torch.cuda.memory_allocated()


def launch_counts():
    """(gemm, memory-bound ops, attention, comm) kernel launches since import."""
    c = _load_ext()
    return tuple(c.launch_counts()) if c is not None else (0, 0, 0, 0)


def affine_cols(a, scale, shift=None):
    """a[r, c] * scale[c] (+ shift[c])."""
    if a.is_cuda:
        return ext().affine_cols(_k(a), _k(scale.to(a.dtype)),
                                 None if shift is None else _k(shift.to(a.dtype)))
    out = a * scale.reshape(1, -1)
    return out if shift is None else out + shift.reshape(1, -1)


# ------------------------------------------------------------------------------ attention (4-d)
def _bgemm(a, b, c, M, N, K, lda, ldb, ldc, a_mn, b_mn, H, Bn, a_s, b_s, c_s, alpha=1.0, causal=0):
    ext().gemm(a, b, c, M, N, K, lda, ldb, ldc, a_mn, b_mn, H, Bn, a_s[0], a_s[1], b_s[0], b_s[1],
               c_s[0], c_s[1], alpha, False, None, 0, None, 0, None, None, 0, causal)


def _attn_composed_forward(q, k, v, causal, scale):
    """Attention for head sizes the flash kernel does not cover: batched tensor-core GEMMs
    plus the score-softmax kernel, scores materialised as [B, H, S, S] bf16."""
    Bn, S, H, D = q.shape
    p = torch.empty((Bn, H, S, S), device=q.device, dtype=torch.bfloat16)
    _bgemm(q, k, p, S, S, D, q.stride(1), k.stride(1), S, False, False, H, Bn,
           (q.stride(2), q.stride(0)), (k.stride(2), k.stride(0)), (S * S, H * S * S), scale,
           1 if causal else 0)
    ext().softmax_scores(p, Bn * H, S, S, causal)
    o = torch.empty((Bn, S, H, D), device=q.device, dtype=torch.bfloat16)
    _bgemm(p, v, o, S, D, S, S, v.stride(1), H * D, False, True, H, Bn, (S * S, H * S * S),
           (v.stride(2), v.stride(0)), (D, S * H * D))
    return o, p


def _attn_composed_backward(q, k, v, p, d_o, causal, scale, dq, dk, dv):
    Bn, S, H, D = q.shape
    ps = (S * S, H * S * S)
    _bgemm(p, d_o, dv, S, D, S, S, d_o.stride(1), dv.stride(1), True, True, H, Bn, ps,
           (d_o.stride(2), d_o.stride(0)), (dv.stride(2), dv.stride(0)))
    dp = torch.empty_like(p)
    _bgemm(d_o, v, dp, S, S, D, d_o.stride(1), v.stride(1), S, False, False, H, Bn,
           (d_o.stride(2), d_o.stride(0)), (v.stride(2), v.stride(0)), ps, 1.0, 1 if causal else 0)
    ext().softmax_scores_backward(p, dp, S, scale, causal)
    _bgemm(dp, k, dq, S, D, S, S, k.stride(1), dq.stride(1), False, True, H, Bn, ps,
           (k.stride(2), k.stride(0)), (dq.stride(2), dq.stride(0)))
    _bgemm(dp, q, dk, S, D, S, S, q.stride(1), dk.stride(1), True, True, H, Bn, ps,
           (q.stride(2), q.stride(0)), (dk.stride(2), dk.stride(0)))


def attention_forward(q, k, v, causal: bool, scale: float):
    """q, k, v: [B, S, H, D] views (unit stride on D). Returns (o [B, S, H, D], ctx)."""
    D = q.shape[-1]
    if q.is_cuda:
        if q.dtype != torch.bfloat16:
            q, k, v = (t.to(torch.bfloat16) for t in (q, k, v))
        if D in (64, 128):
            o, lse = ext().flash_forward(q, k, v, causal, scale)
            if _debug._on:
                _debug.check_kernels(ext())
            return o, ("flash", lse)
        o, p = _attn_composed_forward(q, k, v, causal, scale)
        return o, ("composed", p)
    qh, kh, vh = (t.float().permute(0, 2, 1, 3) for t in (q, k, v))
    s = torch.matmul(qh, kh.transpose(-1, -2)) * scale
    if causal:
        S = q.shape[1]
        s = s.masked_fill(torch.triu(torch.ones(S, S, dtype=torch.bool), 1), -math.inf)
    p = torch.softmax(s, -1)
    o = torch.matmul(p, vh).permute(0, 2, 1, 3).contiguous().to(q.dtype)
    return o, ("cpu", p)


def attention_backward(q, k, v, o, ctx, d_o, causal: bool, scale: float, packed_out=None):
    """Returns (dq, dk, dv) as [B, S, H, D]; with `packed_out` ([B, S, 3, H, D]) the three
    gradients are written into it (the layout of a fused QKV activation)."""
    kind, saved = ctx
    if kind == "cpu":
        p = saved
        qh, kh, vh, doh = (t.float().permute(0, 2, 1, 3) for t in (q, k, v, d_o))
        dv = torch.matmul(p.transpose(-1, -2), doh)
        dp = torch.matmul(doh, vh.transpose(-1, -2))
        ds = p * (dp - (dp * p).sum(-1, keepdim=True)) * scale
        dq = torch.matmul(ds, kh)
        dk = torch.matmul(ds.transpose(-1, -2), qh)
        outs = [t.permute(0, 2, 1, 3).contiguous().to(q.dtype) for t in (dq, dk, dv)]
        if packed_out is not None:
            for i, t in enumerate(outs):
                packed_out[:, :, i].copy_(t)
        return outs
    if q.dtype != torch.bfloat16:
        q, k, v = (t.to(torch.bfloat16) for t in (q, k, v))
    d_o = d_o if d_o.dtype == torch.bfloat16 else d_o.to(torch.bfloat16)
    if d_o.stride(-1) != 1:
        d_o = d_o.contiguous()
    if kind == "flash":
        grads = ext().flash_backward(q, k, v, o, saved, d_o, causal, scale, packed_out)
        if _debug._on:
            _debug.check_kernels(ext())
        return grads
    Bn, S, H, D = q.shape
    if packed_out is not None:
        dq, dk, dv = packed_out[:, :, 0], packed_out[:, :, 1], packed_out[:, :, 2]
    else:
        dq, dk, dv = (torch.empty((Bn, S, H, D), device=q.device, dtype=torch.bfloat16) for _ in range(3))
    _attn_composed_backward(q, k, v, saved, d_o, causal, scale, dq, dk, dv)
    return [dq, dk, dv]
