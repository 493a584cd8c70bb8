"""Binary checkpoints, byte-compatible with the reference's `lf.io.checkpoint`
(lua/luatorch/io/checkpoint.lua:26-115).

File layout (little-endian, exactly what the reference's string.pack calls emit):

    int32  n_params
    n_params records, in model.parameters() order:
        int32  ndim
        int32  dtype_code      0 float32, 1 float64, 2 int32, 3 int64  (float16 / bfloat16 -> 0)
        int64  shape[ndim]
        <elem> data[numel]     row-major

`save` / `load` move whole tensors (one numpy view per parameter) instead of the reference's
per-element Lua loop, check count / ndim / every dimension with the same error messages, and
work for CUDA-resident and arena-backed parameters (the fp32 master copy is what is saved;
bf16 shadows are refreshed after a load).

The reference saves nothing but parameters, so a run cannot really be resumed.
`save_training_state` / `load_training_state` add sidecar files next to the `.bin`
(`<path>.opt.bin` in the same record format + `<path>.state.json`) holding optimizer moments,
step counters, scheduler / GradScaler state, RNG state and module buffers such as BatchNorm
running statistics; the `.bin` itself is untouched by this extension.
"""
from __future__ import annotations

import json
import os
import struct
from typing import List, Optional

import numpy as np
import torch

from .. import _backend as B
from ..tensor import Tensor

_DTYPE_CODE = {torch.float32: 0, torch.float64: 1, torch.int32: 2, torch.int64: 3}
_CODE_NP = {0: np.dtype("<f4"), 1: np.dtype("<f8"), 2: np.dtype("<i4"), 3: np.dtype("<i8")}
_CODE_TORCH = {0: torch.float32, 1: torch.float64, 2: torch.int32, 3: torch.int64}


def _write_record(f, t: torch.Tensor) -> None:
    t = t.detach()
    code = _DTYPE_CODE.get(t.dtype, 0)
    if t.dtype not in _DTYPE_CODE:
        t = t.float()
    arr = t.cpu().contiguous().numpy().astype(_CODE_NP[code], copy=False)
    f.write(struct.pack("<i", t.dim()))
    f.write(struct.pack("<i", code))
    for s in t.shape:
        f.write(struct.pack("<q", int(s)))
    f.write(arr.tobytes(order="C"))


def _read_record(f):
    ndim = struct.unpack("<i", f.read(4))[0]
    raw = f.read(4)
    code = struct.unpack("<i", raw)[0] if len(raw) == 4 else 0
    if code not in _CODE_NP:
        code = 0
    shape = [struct.unpack("<q", f.read(8))[0] for _ in range(ndim)]
    n = 1
    for s in shape:
        n *= s
    dt = _CODE_NP[code]
    buf = f.read(n * dt.itemsize)
    if len(buf) != n * dt.itemsize:
        raise IOError("luatorch error: checkpoint file is truncated")
    arr = np.frombuffer(buf, dtype=dt).reshape(shape) if n else np.zeros(shape, dtype=dt)
    return ndim, shape, torch.from_numpy(arr.copy())


def save(model, path: str) -> None:
    params: List[Tensor] = model.parameters()
    try:
        f = open(path, "wb")
    except OSError:
        raise IOError("luatorch error: could not open file for writing: " + path)
    with f:
        f.write(struct.pack("<i", len(params)))
        for p in params:
            _write_record(f, p._t)


def load(model, path: str) -> None:
    params: List[Tensor] = model.parameters()
    try:
        f = open(path, "rb")
    except OSError:
        raise IOError("luatorch error: could not open file for reading: " + path)
    with f:
        n_params = struct.unpack("<i", f.read(4))[0]
        if n_params != len(params):
            raise ValueError("luatorch error: parameter count mismatch, file has %d but model has %d"
                             % (n_params, len(params)))
        for idx, p in enumerate(params, start=1):
            ndim, shape, data = _read_record(f)
            if ndim != p.ndim:
                raise ValueError("luatorch error: ndim mismatch for parameter %d, file has %d but "
                                 "model has %d" % (idx, ndim, p.ndim))
            for i, (a, b) in enumerate(zip(shape, p.shape), start=1):
                if a != b:
                    raise ValueError("luatorch error: shape mismatch for parameter %d dimension %d"
                                     % (idx, i))
            p._t.copy_(data.to(p._t.dtype))
            if p._compute is not None:
                p._compute.copy_(p._t)


# ------------------------------------------------------------------------------ resume sidecars
def _module_buffers(model) -> List[Tensor]:
    out = []

    def walk(m):
        if hasattr(m, "buffers"):
            out.extend(m.buffers())
        for c in (m.children() if hasattr(m, "children") else []):
            walk(c)

    walk(model)
    return out


def save_training_state(path: str, model=None, optimizer=None, scheduler=None, scaler=None,
                        step: int = 0, extra: Optional[dict] = None,
                        optimizer_state: Optional[dict] = None) -> None:
    """`optimizer_state`: a state_dict() taken beforehand (with state sharded over ranks,
    state_dict() is a collective that every rank has to enter, while only one rank writes)."""
    tensors: List[torch.Tensor] = []
    meta = {"step": int(step), "extra": extra or {}, "format": 1}
    if optimizer is not None:
        sd = optimizer_state if optimizer_state is not None else optimizer.state_dict()
        groups = {}
        for k, v in sd.items():
            if isinstance(v, list) and v and isinstance(v[0], torch.Tensor):
                groups[k] = [len(tensors), len(v)]
                tensors.extend(v)
            else:
                meta.setdefault("optimizer", {})[k] = v
        meta["optimizer_tensors"] = groups
    if model is not None:
        bufs = _module_buffers(model)
        meta["buffers"] = [len(tensors), len(bufs)]
        tensors.extend(b._t for b in bufs)
    if scheduler is not None and hasattr(scheduler, "state_dict"):
        meta["scheduler"] = scheduler.state_dict()
    if scaler is not None and hasattr(scaler, "state_dict"):
        meta["scaler"] = scaler.state_dict()
    rng = B.rng_state()
    meta["rng"] = {"seed": rng["seed"], "offset": rng["offset"]}
    tensors.append(rng["cpu"].clone().to(torch.int32))
    with open(path + ".opt.bin", "wb") as f:
        f.write(struct.pack("<i", len(tensors)))
        for t in tensors:
            _write_record(f, t)
    tmp = path + ".state.json.tmp"
    with open(tmp, "w") as f:
        json.dump(meta, f)
    os.replace(tmp, path + ".state.json")


def load_training_state(path: str, model=None, optimizer=None, scheduler=None, scaler=None) -> dict:
    with open(path + ".state.json") as f:
        meta = json.load(f)
    with open(path + ".opt.bin", "rb") as f:
        n = struct.unpack("<i", f.read(4))[0]
        tensors = [_read_record(f)[2] for _ in range(n)]
    if optimizer is not None and "optimizer_tensors" in meta:
        sd = dict(meta.get("optimizer", {}))
        for k, (start, cnt) in meta["optimizer_tensors"].items():
            sd[k] = tensors[start:start + cnt]
        optimizer.load_state_dict(sd)
    if model is not None and "buffers" in meta:
        start, cnt = meta["buffers"]
        for b, src in zip(_module_buffers(model), tensors[start:start + cnt]):
            b._t.copy_(src.to(b._t.dtype))
    if scheduler is not None and "scheduler" in meta:
        scheduler.load_state_dict(meta["scheduler"])
    if scaler is not None and "scaler" in meta:
        scaler.load_state_dict(meta["scaler"])
    if "rng" in meta:
        B.set_rng_state({"seed": meta["rng"]["seed"], "offset": meta["rng"]["offset"],
                         "cpu": tensors[-1].to(torch.uint8)})
    return meta
