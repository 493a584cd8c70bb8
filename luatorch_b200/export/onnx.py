"""ONNX export without any ONNX dependency: a small protobuf writer plus a module walker.

The reference's exporter writes every parameter as an initializer but its graph is a single
placeholder MatMul node (lua/luatorch/export/onnx.lua:180-188) and `verify` only looks at the
file size and first byte (:244-268).  Here `export(model, dummy_input, path)` emits the real
operator graph of the supported modules (Linear -> MatMul+Add, activations, LayerNorm,
Dropout as Identity, Embedding -> Gather, Sequential / MLP chains, GPT with decomposed
attention), ir_version 7 / opset 13 / producer "luatorch" as in the reference, and
`verify(path)` parses the file back and checks its structure; `run(path, input)` evaluates the
stored graph with numpy (every operator the exporter emits), so an export can be checked
numerically against the model it came from without an ONNX runtime: `verify(path, model, x)`.
"""
from __future__ import annotations

import struct
from typing import Dict, List, Tuple

import numpy as np

from .. import autograd
from ..tensor import Tensor

# ------------------------------------------------------------------------------ protobuf writer


def _varint(n: int) -> bytes:
    if n < 0:
        n += 1 << 64
    out = bytearray()
    while True:
        b = n & 0x7F
        n >>= 7
        if n:
            out.append(b | 0x80)
        else:
            out.append(b)
            return bytes(out)


def _tag(field: int, wire: int) -> bytes:
    return _varint((field << 3) | wire)


def _bytes(field: int, payload: bytes) -> bytes:
    return _tag(field, 2) + _varint(len(payload)) + payload


def _string(field: int, s: str) -> bytes:
    return _bytes(field, s.encode("utf-8"))


def _int(field: int, v: int) -> bytes:
    return _tag(field, 0) + _varint(int(v))


def _float(field: int, v: float) -> bytes:
    return _tag(field, 5) + struct.pack("<f", float(v))


FLOAT, INT64 = 1, 7


def tensor_proto(name: str, arr: np.ndarray) -> bytes:
    out = b""
    for d in arr.shape:
        out += _int(1, d)
    if arr.dtype == np.int64:
        out += _int(2, INT64)
        raw = arr.astype("<i8").tobytes()
    else:
        out += _int(2, FLOAT)
        raw = arr.astype("<f4").tobytes()
    out += _string(8, name)
    out += _bytes(9, raw)          # raw_data
    return out


def attribute(name: str, value) -> bytes:
    out = _string(1, name)
    if isinstance(value, float):
        out += _float(2, value) + _int(20, 1)
    elif isinstance(value, int):
        out += _int(3, value) + _int(20, 2)
    elif isinstance(value, (list, tuple)):
        for v in value:
            out += _int(8, v)
        out += _int(20, 7)
    else:
        raise TypeError(value)
    return out


def node_proto(op: str, inputs: List[str], outputs: List[str], name: str = "", **attrs) -> bytes:
    out = b""
    for i in inputs:
        out += _string(1, i)
    for o in outputs:
        out += _string(2, o)
    if name:
        out += _string(3, name)
    out += _string(4, op)
    for k, v in attrs.items():
        out += _bytes(5, attribute(k, v))
    return out


def value_info(name: str, shape, elem_type: int = FLOAT) -> bytes:
    dims = b""
    for d in shape:
        dims += _bytes(1, _int(1, d))
    tensor_type = _int(1, elem_type) + _bytes(2, dims)
    return _string(1, name) + _bytes(2, _bytes(1, tensor_type))


# ------------------------------------------------------------------------------ graph builder
class _Graph:
    def __init__(self):
        self.nodes: List[bytes] = []
        self.inits: List[bytes] = []
        self.n = 0
        self.n_init = 0
        self.n_params = 0

    def name(self, prefix: str) -> str:
        self.n += 1
        return "%s_%d" % (prefix, self.n)

    def init(self, t, prefix: str = "param") -> str:
        arr = t._t.detach().float().cpu().contiguous().numpy() if isinstance(t, Tensor) else np.asarray(t)
        self.n_init += 1
        nm = "%s_%d" % (prefix, self.n_init)
        self.inits.append(tensor_proto(nm, arr))
        if isinstance(t, Tensor):
            self.n_params += arr.size
        return nm

    def const_i64(self, values) -> str:
        return self.init(np.asarray(values, dtype=np.int64), "const")

    def op(self, op: str, inputs: List[str], prefix: str = "t", **attrs) -> str:
        out = self.name(prefix)
        self.nodes.append(node_proto(op, inputs, [out], self.name(op), **attrs))
        return out


def _emit(g: _Graph, m, x: str, ctx: dict) -> str:
    from .. import nn
    from ..models.gpt import GPT
    from ..models.mlp import MLP
    if isinstance(m, nn.Sequential):
        for layer in m.layers:
            x = _emit(g, layer, x, ctx)
        return x
    if isinstance(m, MLP):
        return _emit(g, m.net, x, ctx)
    if isinstance(m, nn.Linear):
        y = g.op("MatMul", [x, g.init(m.weight)])
        return g.op("Add", [y, g.init(m.bias)]) if m.use_bias else y
    if isinstance(m, nn.ReLU):
        return g.op("Relu", [x])
    if isinstance(m, nn.Sigmoid):
        return g.op("Sigmoid", [x])
    if isinstance(m, nn.Tanh):
        return g.op("Tanh", [x])
    if isinstance(m, nn.SiLU):
        return g.op("Mul", [x, g.op("Sigmoid", [x])])
    if isinstance(m, nn.GELU):
        # tanh approximation: 0.5 x (1 + tanh(k0 (x + k1 x^3)))
        x3 = g.op("Mul", [g.op("Mul", [x, x]), x])
        inner = g.op("Add", [x, g.op("Mul", [x3, g.init(np.float32(0.044715), "const")])])
        t = g.op("Tanh", [g.op("Mul", [inner, g.init(np.float32(0.7978845608), "const")])])
        half = g.op("Mul", [x, g.init(np.float32(0.5), "const")])
        return g.op("Mul", [half, g.op("Add", [t, g.init(np.float32(1.0), "const")])])
    if isinstance(m, nn.Dropout):
        return g.op("Identity", [x])
    if isinstance(m, nn.LayerNorm):
        mean = g.op("ReduceMean", [x], axes=[-1], keepdims=1)
        xc = g.op("Sub", [x, mean])
        var = g.op("ReduceMean", [g.op("Mul", [xc, xc])], axes=[-1], keepdims=1)
        std = g.op("Sqrt", [g.op("Add", [var, g.init(np.float32(m.eps), "const")])])
        y = g.op("Mul", [g.op("Div", [xc, std]), g.init(m.gamma)])
        return g.op("Add", [y, g.init(m.beta)])
    if isinstance(m, nn.BatchNorm1d):
        rstd = 1.0 / np.sqrt(m.running_var._t.float().cpu().numpy() + m.eps)
        scale = m.gamma._t.detach().float().cpu().numpy() * rstd
        shift = m.beta._t.detach().float().cpu().numpy() - m.running_mean._t.float().cpu().numpy() * scale
        return g.op("Add", [g.op("Mul", [x, g.init(scale, "const")]), g.init(shift, "const")])
    if isinstance(m, nn.Embedding):
        return g.op("Gather", [g.init(m.weight), x], axis=0)
    if isinstance(m, nn.MultiHeadAttention):
        S, Bn, H, D = ctx["seq_len"], ctx["batch"], m.num_heads, m.head_dim
        def heads(t):
            r = g.op("Reshape", [t, g.const_i64([Bn, S, H, D])])
            return g.op("Transpose", [r], perm=[0, 2, 1, 3])
        q = heads(g.op("MatMul", [x, g.init(m.q_proj.weight)]))
        k = heads(g.op("MatMul", [x, g.init(m.k_proj.weight)]))
        v = heads(g.op("MatMul", [x, g.init(m.v_proj.weight)]))
        s = g.op("MatMul", [q, g.op("Transpose", [k], perm=[0, 1, 3, 2])])
        s = g.op("Mul", [s, g.init(np.float32(m.scale), "const")])
        if m.causal:
            mask = np.triu(np.full((S, S), -1e9, dtype=np.float32), 1)
            s = g.op("Add", [s, g.init(mask, "const")])
        p = g.op("Softmax", [s], axis=-1)
        o = g.op("Transpose", [g.op("MatMul", [p, v])], perm=[0, 2, 1, 3])
        o = g.op("Reshape", [o, g.const_i64([Bn * S, H * D])])
        return _emit(g, m.out_proj, o, ctx)
    if isinstance(m, nn.TransformerBlock):
        a = _emit(g, m.attn, _emit(g, m.ln1, x, ctx), ctx)
        x = g.op("Add", [x, a])
        h = _emit(g, m.ffn1, _emit(g, m.ln2, x, ctx), ctx)
        h = _emit(g, m.ffn2, _emit(g, m.gelu, h, ctx), ctx)
        return g.op("Add", [x, h])
    if isinstance(m, GPT):
        S, Bn = ctx["seq_len"], ctx["batch"]
        ids = g.op("Reshape", [g.op("Cast", [x], to=INT64), g.const_i64([Bn * S])])
        h = g.op("Gather", [g.init(m.token_emb.weight), ids], axis=0)
        table = m.pos_enc.weight if hasattr(m.pos_enc, "weight") else m.pos_enc.pe
        pos = table._t.detach().float().cpu().numpy()[:S]
        pe = g.init(np.tile(pos, (Bn, 1)), "param" if hasattr(m.pos_enc, "weight") else "const")
        h = g.op("Add", [h, pe])
        for b in m.blocks:
            h = _emit(g, b, h, ctx)
        return _emit(g, m.head, _emit(g, m.final_ln, h, ctx), ctx)
    raise TypeError("onnx export: unsupported module %r" % (m,))


def export(model, dummy_input: Tensor, path: str) -> None:
    with autograd.no_grad():
        out = model(dummy_input)
    out = out[0] if isinstance(out, tuple) else out
    g = _Graph()
    shape = dummy_input.shape
    ctx = {"batch": shape[0] if len(shape) >= 2 else 1, "seq_len": shape[1] if len(shape) >= 2 else shape[0]}
    y = _emit(g, getattr(model, "model", model), "input_1", ctx)
    g.nodes.append(node_proto("Identity", [y], ["output_1"], "output"))
    graph = b"".join(_bytes(1, n) for n in g.nodes) + _string(2, "luatorch_model")
    graph += b"".join(_bytes(5, t) for t in g.inits)
    graph += _bytes(11, value_info("input_1", shape)) + _bytes(12, value_info("output_1", out.shape))
    model_proto = _int(1, 7) + _string(2, "luatorch") + _bytes(7, graph) + _bytes(8, _string(1, "") + _int(2, 13))
    try:
        f = open(path, "wb")
    except OSError:
        raise IOError("luatorch error: could not open %s for writing" % path)
    with f:
        f.write(model_proto)
    print("exported onnx model to %s (%d parameters, %d initializers, %d nodes)" % (
        path, g.n_params, len(g.inits), len(g.nodes)))


# ------------------------------------------------------------------------------ reader / verify
def _read_varint(buf: bytes, pos: int) -> Tuple[int, int]:
    n = shift = 0
    while True:
        b = buf[pos]
        pos += 1
        n |= (b & 0x7F) << shift
        if not b & 0x80:
            return n, pos
        shift += 7


def _fields(buf: bytes):
    pos = 0
    while pos < len(buf):
        key, pos = _read_varint(buf, pos)
        field, wire = key >> 3, key & 7
        if wire == 0:
            v, pos = _read_varint(buf, pos)
        elif wire == 2:
            ln, pos = _read_varint(buf, pos)
            v = buf[pos:pos + ln]
            pos += ln
        elif wire == 5:
            v = buf[pos:pos + 4]
            pos += 4
        elif wire == 1:
            v = buf[pos:pos + 8]
            pos += 8
        else:
            raise ValueError("bad wire type %d" % wire)
        yield field, wire, v


def inspect(path: str) -> Dict:
    """Parse an exported file: ir version, producer, opset, op list, initializer names."""
    with open(path, "rb") as f:
        buf = f.read()
    info = {"ir_version": None, "producer": None, "opset": None, "ops": [], "initializers": [],
            "inputs": [], "outputs": []}
    for field, wire, v in _fields(buf):
        if field == 1 and wire == 0:
            info["ir_version"] = v
        elif field == 2 and wire == 2:
            info["producer"] = v.decode()
        elif field == 8 and wire == 2:
            for f2, w2, v2 in _fields(v):
                if f2 == 2:
                    info["opset"] = v2
        elif field == 7 and wire == 2:
            for f2, w2, v2 in _fields(v):
                if f2 == 1:
                    info["ops"].append(next(x.decode() for ff, ww, x in _fields(v2) if ff == 4))
                elif f2 == 5:
                    info["initializers"].append(next(x.decode() for ff, ww, x in _fields(v2) if ff == 8))
                elif f2 in (11, 12):
                    nm = next(x.decode() for ff, ww, x in _fields(v2) if ff == 1)
                    info["inputs" if f2 == 11 else "outputs"].append(nm)
    return info


def _signed(v: int) -> int:
    return v - (1 << 64) if v >= 1 << 63 else v


def load_graph(path: str) -> Dict:
    """Full parse: {"nodes": [(op, inputs, outputs, attrs)], "initializers": {name: ndarray},
    "input": name, "output": name}."""
    with open(path, "rb") as f:
        buf = f.read()
    graph = next(v for field, wire, v in _fields(buf) if field == 7 and wire == 2)
    nodes, inits, g_in, g_out = [], {}, None, None
    for f2, w2, v2 in _fields(graph):
        if f2 == 1:
            ins, outs, op, attrs = [], [], None, {}
            for ff, ww, x in _fields(v2):
                if ff == 1:
                    ins.append(x.decode())
                elif ff == 2:
                    outs.append(x.decode())
                elif ff == 4:
                    op = x.decode()
                elif ff == 5:
                    name, val, ints = None, None, []
                    for fa, wa, xa in _fields(x):
                        if fa == 1:
                            name = xa.decode()
                        elif fa == 2:
                            val = struct.unpack("<f", xa)[0]
                        elif fa == 3:
                            val = _signed(xa)
                        elif fa == 8:
                            ints.append(_signed(xa))
                    attrs[name] = ints if ints else val
            nodes.append((op, ins, outs, attrs))
        elif f2 == 5:
            dims, dtype, name, raw = [], FLOAT, None, b""
            for ff, ww, x in _fields(v2):
                if ff == 1:
                    dims.append(x)
                elif ff == 2:
                    dtype = x
                elif ff == 8:
                    name = x.decode()
                elif ff == 9:
                    raw = x
            inits[name] = np.frombuffer(raw, dtype="<i8" if dtype == INT64 else "<f4").reshape(dims)
        elif f2 in (11, 12):
            nm = next(x.decode() for ff, ww, x in _fields(v2) if ff == 1)
            if f2 == 11:
                g_in = nm
            else:
                g_out = nm
    return {"nodes": nodes, "initializers": inits, "input": g_in, "output": g_out}


def _softmax(x: np.ndarray, axis: int) -> np.ndarray:
    e = np.exp(x - x.max(axis=axis, keepdims=True))
    return e / e.sum(axis=axis, keepdims=True)


_NUMPY_OPS = {
    "MatMul": lambda a, i: np.matmul(i[0], i[1]),
    "Add": lambda a, i: i[0] + i[1],
    "Sub": lambda a, i: i[0] - i[1],
    "Mul": lambda a, i: i[0] * i[1],
    "Div": lambda a, i: i[0] / i[1],
    "Sqrt": lambda a, i: np.sqrt(i[0]),
    "Relu": lambda a, i: np.maximum(i[0], 0),
    "Sigmoid": lambda a, i: 1.0 / (1.0 + np.exp(-i[0])),
    "Tanh": lambda a, i: np.tanh(i[0]),
    "Identity": lambda a, i: i[0],
    "ReduceMean": lambda a, i: i[0].mean(axis=tuple(a["axes"]), keepdims=bool(a.get("keepdims", 1))),
    "Gather": lambda a, i: np.take(i[0], i[1].astype(np.int64), axis=a.get("axis", 0)),
    "Reshape": lambda a, i: i[0].reshape([int(d) for d in i[1]]),
    "Transpose": lambda a, i: np.transpose(i[0], a["perm"]),
    "Softmax": lambda a, i: _softmax(i[0], a.get("axis", -1)),
    "Cast": lambda a, i: i[0].astype(np.int64 if a["to"] == INT64 else np.float32),
}


def run(path: str, input) -> np.ndarray:
    """Evaluate an exported file on `input` (Tensor, torch tensor or array) with numpy."""
    g = load_graph(path)
    if isinstance(input, Tensor):
        input = input._t
    if hasattr(input, "detach"):
        input = input.detach().float().cpu().numpy()
    env = dict(g["initializers"])
    env[g["input"]] = np.asarray(input, dtype=np.float32)
    for op, ins, outs, attrs in g["nodes"]:
        fn = _NUMPY_OPS.get(op)
        if fn is None:
            raise NotImplementedError("onnx run: operator %s" % op)
        env[outs[0]] = fn(attrs, [env[n] for n in ins])
    return env[g["output"]]


def verify(path: str, model=None, dummy_input=None, tol: float = 1e-4) -> bool:
    """Structure check; with `model` and `dummy_input` also a numeric check of the stored graph
    (numpy evaluation) against the model's own forward."""
    try:
        info = inspect(path)
    except Exception as e:
        print("onnx verify: cannot parse %s: %r" % (path, e))
        return False
    ok = (info["ir_version"] == 7 and info["opset"] == 13 and info["producer"] == "luatorch"
          and len(info["ops"]) > 0 and len(info["inputs"]) == 1 and len(info["outputs"]) == 1)
    if ok and model is not None and dummy_input is not None:
        with autograd.no_grad():
            want = model(dummy_input)
        want = (want[0] if isinstance(want, tuple) else want)._t.detach().float().cpu().numpy()
        got = run(path, dummy_input).reshape(want.shape)
        err = float(np.abs(got - want).max())
        ok = err <= tol * max(1.0, float(np.abs(want).max()))
        print("onnx numeric check: max abs error %.3g (%s)" % (err, "ok" if ok else "MISMATCH"))
    print("onnx file %s: %s (%d nodes, %d initializers)" % (
        path, "valid" if ok else "INVALID", len(info["ops"]), len(info["initializers"])))
    return ok
