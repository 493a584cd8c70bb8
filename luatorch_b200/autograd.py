"""Tape autograd with the reference's surface: watch / record / backward / zero_graph /
zero_grad / acc_grad / enabled / graph and the tracked ops add, mul, matmul, relu
(lua/luatorch/autograd.lua:18-169).

Same model: a flat list of nodes in creation order, walked in reverse; each node owns a
closure that pushes gradients into its inputs.  Differences that matter on a GPU:
  * the seed gradient lives on the loss's device (the reference seeds a CPU tensor, :138-142);
  * parameters that own a preallocated gradient buffer (`Tensor._grad_buf`, set by the
    parameter arena) receive gradients in place, so the bucketed all-reduce can start as soon
    as the last contribution lands;
  * a per-leaf use count tells when a parameter's gradient is final and fires its hook;
  * `no_grad()` context manager in addition to the `enabled` flag.
"""
from __future__ import annotations

from contextlib import contextmanager
from typing import Callable, List, Optional, Sequence

import torch

from . import _backend as B
from .tensor import Tensor


class Node:
    __slots__ = ("tensor", "op", "parents", "grad_fn")

    def __init__(self, tensor, op, parents=None):
        self.tensor = tensor
        self.op = op
        self.parents = parents or []
        self.grad_fn: Optional[Callable] = None


enabled = True
graph: List[Node] = []
_pending_uses = {}   # id(leaf tensor) -> [tensor, outstanding uses]


def zero_graph() -> None:
    """Drop the tape.  Nodes and their closures reference each other through the tensors
    they produced (tensor._node -> node.grad_fn -> tensor); the links are cut here so the
    activations are released by reference counting at once instead of waiting for the cycle
    collector (which otherwise lets device memory pile up across steps)."""
    global graph
    for node in graph:
        t = node.tensor
        if t is not None and t._node is node:
            t._node = None
        node.grad_fn = None
        node.parents = ()
        node.tensor = None
    graph = []
    _pending_uses.clear()


def watch(tensor: Tensor) -> Tensor:
    tensor.requires_grad = True
    tensor.grad = None
    tensor._node = Node(tensor, "leaf", [])
    return tensor


def record(op: str, inputs: Sequence[Tensor], output: Tensor, grad_fn: Callable) -> None:
    if not enabled:
        return
    needs = False
    for inp in inputs:
        if inp is not None and inp.requires_grad:
            needs = True
            if inp._hook is not None:
                slot = _pending_uses.get(id(inp))
                if slot is None:
                    _pending_uses[id(inp)] = [inp, 1]
                else:
                    slot[1] += 1
    if needs:
        output.requires_grad = True
    node = Node(output, op, list(inputs))
    node.grad_fn = grad_fn
    output._node = node
    graph.append(node)


def acc_grad(tensor: Tensor, new_grad) -> None:
    """Accumulate `new_grad` (Tensor or torch.Tensor) into tensor.grad."""
    g = new_grad._t if isinstance(new_grad, Tensor) else new_grad
    if tensor._grad_buf is not None:
        buf = tensor._grad_buf
        if tensor.grad is None:
            if g.data_ptr() != buf.data_ptr():
                buf.copy_(g.reshape(buf.shape))
            tensor.grad = Tensor(_data=buf)
        else:
            B.binary_inplace("add", buf, g.reshape(buf.shape).to(buf.dtype))
        return
    if tensor.grad is not None:
        tensor.grad = Tensor(_data=B.binary("add", tensor.grad._t, g.reshape(tensor.grad._t.shape)))
    else:
        tensor.grad = Tensor(_data=g.reshape(tensor._t.shape) if g.numel() == tensor._t.numel() else g)


def grad_target(tensor: Tensor):
    """For kernels that can write a parameter gradient in place: returns (buffer, accumulate)
    or (None, False) when the tensor has no preallocated gradient storage."""
    if tensor._grad_buf is None:
        return None, False
    return tensor._grad_buf, tensor.grad is not None


def grad_written(tensor: Tensor) -> None:
    """Declare that `grad_target(tensor)[0]` now holds the (accumulated) gradient."""
    if tensor.grad is None:
        tensor.grad = Tensor(_data=tensor._grad_buf)


def _leaf_done(node: Node) -> None:
    for inp in node.parents:
        if inp is None or inp._hook is None:
            continue
        slot = _pending_uses.get(id(inp))
        if slot is None:
            continue
        slot[1] -= 1
        if slot[1] == 0:
            del _pending_uses[id(inp)]
            inp._hook(inp)


def backward(loss: Tensor, grad: Optional[Tensor] = None) -> None:
    from .utils import nvtx
    with nvtx.range("autograd.backward"):
        _backward(loss, grad)


def _backward(loss: Tensor, grad: Optional[Tensor] = None) -> None:
    if grad is None:
        seed = torch.ones_like(loss._t)
    else:
        seed = grad._t if isinstance(grad, Tensor) else grad
    loss.grad = Tensor(_data=seed)
    loss.grad._unit = grad is None
    for i in range(len(graph) - 1, -1, -1):
        node = graph[i]
        if node.grad_fn is not None and node.tensor.grad is not None:
            node.grad_fn(node.tensor.grad)
            # intermediates drop their gradient once consumed (peak memory, as the
            # reference does in autograd.lua:149-156); leaves keep theirs
            if node.op != "leaf":
                node.tensor.grad = None
            if _pending_uses:
                _leaf_done(node)
            # the closure holds the activations saved for this node: release them now
            node.grad_fn = None
            node.parents = ()


def zero_grad(tensors: Sequence[Tensor]) -> None:
    for t in tensors:
        t.grad = None


@contextmanager
def no_grad():
    global enabled
    prev = enabled
    enabled = False
    try:
        yield
    finally:
        enabled = prev


def set_enabled(flag: bool) -> None:
    global enabled
    enabled = bool(flag)


# ------------------------------------------------------------------------------ tracked ops
def add(a: Tensor, b: Tensor) -> Tensor:
    out = Tensor.add(a, b)

    def grad_fn(g):
        if a.requires_grad:
            acc_grad(a, g)
        if b.requires_grad:
            acc_grad(b, g)

    record("add", [a, b], out, grad_fn)
    return out


def mul(a: Tensor, b: Tensor) -> Tensor:
    out = Tensor.mul(a, b)

    def grad_fn(g):
        if a.requires_grad:
            acc_grad(a, Tensor.mul(g, b))
        if b.requires_grad:
            acc_grad(b, Tensor.mul(g, a))

    record("mul", [a, b], out, grad_fn)
    return out


def matmul(a: Tensor, b: Tensor) -> Tensor:
    out = Tensor.matmul(a, b)

    def grad_fn(g):
        # On CUDA bf16 the transposed products run directly on the tensor cores (operand
        # layout flags), no transposed copy is made.
        if a.requires_grad:
            if g.device == "cuda" and g._t.dtype == torch.bfloat16:
                acc_grad(a, B.gemm(g._t, b._t, b_t=True))
            else:
                acc_grad(a, Tensor.matmul(g, Tensor.transpose(b)))
        if b.requires_grad:
            if g.device == "cuda" and g._t.dtype == torch.bfloat16:
                acc_grad(b, B.gemm(a._t, g._t, a_t=True))
            else:
                acc_grad(b, Tensor.matmul(Tensor.transpose(a), g))

    record("matmul", [a, b], out, grad_fn)
    return out


def relu(x: Tensor) -> Tensor:
    out = Tensor.relu(x)

    def grad_fn(g):
        if x.requires_grad:
            acc_grad(x, B.unary_backward("relu", x._t, g._t))

    record("relu", [x], out, grad_fn)
    return out
