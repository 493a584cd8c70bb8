"""Reference arm of bench.py: the UNMODIFIED reference library (built from the reference
sources with CMake into baseline/_ref/libluatorch.so, `-DLUATORCH_USE_NCCL=ON
-DCMAKE_CUDA_ARCHITECTURES=100`) driven through its own C ABI, the surface its LuaJIT front
end binds (lua/luatorch/tensor.lua:33-178, lua/luatorch/distributed/init.lua:17-21).  LuaJIT
is not installed here, so the Lua layer itself cannot run; and even with it the reference's
model code could not keep a GPT on the GPU (its layers read tensors element by element on the
host).  This harness therefore issues, per training step, the sequence of reference GPU ops a
GPU-resident luatorch GPT step consists of, in fp32 as the reference computes:

  tensor_fused_layernorm_cuda, tensor_matmul_cuda (cuBLAS SGEMM), tensor_flash_attention_cuda,
  tensor_add_broadcast_cuda, tensor_add_cuda, tensor_fused_gelu_bias_cuda,
  tensor_cross_entropy_loss[_backward]_cuda, tensor_transpose_cuda + tensor_matmul_cuda for
  every matmul backward (lua/luatorch/autograd.lua:105-114), tensor_add_broadcast_backward_cuda,
  tensor_fused_adam_cuda once per parameter, luatorch_nccl_allreduce once per parameter
  (lua/luatorch/distributed/ddp.lua:48-61), all devices driven by ONE process as the
  reference's NCCL wrapper requires (csrc/distributed/nccl_wrapper.cu:37-111).

Ops the reference has NO GPU kernel for (LayerNorm / GELU / attention backward, embedding
gather / scatter) are stood in for by the cheapest reference ops of the same tensor shapes
(elementwise passes; bmm + softmax for the attention backward).  That UNDER-counts the
reference's work, so the throughput printed here is an upper bound on what the reference could
reach; none of this repository's kernels or engine are used on this path.
"""
from __future__ import annotations

import ctypes as C
import json
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "_ref", "libluatorch.so")


class RefTensor(C.Structure):
    _fields_ = [("data", C.c_void_p), ("cuda_data", C.c_void_p), ("shape", C.POINTER(C.c_int64)),
                ("strides", C.POINTER(C.c_int64)), ("ndim", C.c_int), ("numel", C.c_int64),
                ("dtype", C.c_int), ("device", C.c_int), ("requires_grad", C.c_int),
                ("grad", C.c_void_p), ("ref_count", C.c_int)]


TP = C.POINTER(RefTensor)


def _load():
    lib = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)
    unary = ["tensor_transpose_cuda", "tensor_softmax_cuda", "tensor_add_broadcast_backward_cuda",
             "tensor_to_cuda", "tensor_tanh_cuda", "tensor_copy"]
    binary = ["tensor_matmul_cuda", "tensor_bmm_cuda", "tensor_add_cuda", "tensor_mul_cuda",
              "tensor_sub_cuda", "tensor_add_broadcast_cuda", "tensor_fused_gelu_bias_cuda",
              "tensor_cross_entropy_loss_cuda", "tensor_cross_entropy_loss_backward_cuda"]
    for n in unary:
        getattr(lib, n).restype, getattr(lib, n).argtypes = TP, [TP]
    for n in binary:
        getattr(lib, n).restype, getattr(lib, n).argtypes = TP, [TP, TP]
    lib.tensor_new.restype, lib.tensor_new.argtypes = TP, [C.POINTER(C.c_int64), C.c_int, C.c_int, C.c_int]
    lib.tensor_new_cuda.restype, lib.tensor_new_cuda.argtypes = TP, [C.POINTER(C.c_int64), C.c_int, C.c_int]
    lib.tensor_reshape.restype, lib.tensor_reshape.argtypes = TP, [TP, C.POINTER(C.c_int64), C.c_int]
    lib.tensor_free.restype, lib.tensor_free.argtypes = None, [TP]
    lib.tensor_randn.restype, lib.tensor_randn.argtypes = None, [TP]
    lib.tensor_fill.restype, lib.tensor_fill.argtypes = None, [TP, C.c_float]
    lib.tensor_set.restype, lib.tensor_set.argtypes = None, [TP, C.c_int64, C.c_float]
    lib.tensor_mul_scalar_cuda_.restype, lib.tensor_mul_scalar_cuda_.argtypes = None, [TP, C.c_float]
    lib.tensor_fused_layernorm_cuda.restype = TP
    lib.tensor_fused_layernorm_cuda.argtypes = [TP, TP, TP, C.c_float]
    lib.tensor_fused_adam_cuda.restype = None
    lib.tensor_fused_adam_cuda.argtypes = [TP, TP, TP, TP] + [C.c_float] * 7
    lib.tensor_flash_attention_cuda.restype = TP
    lib.tensor_flash_attention_cuda.argtypes = [TP, TP, TP, C.c_int, C.c_int, C.c_int, C.c_int]
    lib.tensor_sum_cuda.restype, lib.tensor_sum_cuda.argtypes = C.c_float, [TP]
    lib.pool_init.restype = None
    lib.pool_clear.restype = None

    def _non_null(name):
        def check(result, func, args):
            if not result:
                raise RuntimeError("reference op %s returned NULL (it printed its own error above)" % name)
            return result
        return check

    for n in unary + binary + ["tensor_new", "tensor_new_cuda", "tensor_reshape",
                               "tensor_fused_layernorm_cuda", "tensor_flash_attention_cuda"]:
        getattr(lib, n).errcheck = _non_null(n)
    lib.luatorch_nccl_init.restype, lib.luatorch_nccl_init.argtypes = C.c_int, [C.c_int]
    lib.luatorch_nccl_allreduce.restype = C.c_int
    lib.luatorch_nccl_allreduce.argtypes = [C.POINTER(C.c_void_p), C.c_int64, C.c_int]
    lib.luatorch_nccl_destroy.restype = None
    return lib


class Replica:
    """Weights, optimizer state and one training step of the GPT on ONE device."""

    def __init__(self, lib, rt, dev, cfg, seed_tokens):
        self.lib, self.rt, self.dev, self.cfg = lib, rt, dev, cfg
        rt.cudaSetDevice(dev)
        E, V, L, S, Bm = cfg["embed"], cfg["vocab"], cfg["layers"], cfg["seq"], cfg["micro_batch"]
        self.T = Bm * S
        self.params = []

        def weight(shape, std):
            t = self.cpu(shape)
            lib.tensor_randn(t)
            lib.tensor_to_cuda(t)
            lib.tensor_mul_scalar_cuda_(t, std)
            return self._reg(t)

        def const(shape, val):
            t = self.cpu(shape)
            lib.tensor_fill(t, val)
            lib.tensor_to_cuda(t)
            return self._reg(t)

        self.emb = weight([V, E], 0.02)
        self.pos = weight([S, E], 0.02)
        self.layers = []
        for _ in range(L):
            self.layers.append(dict(
                g1=const([E], 1.0), b1=const([E], 0.0),
                wq=weight([E, E], (2.0 / E) ** 0.5), wk=weight([E, E], (2.0 / E) ** 0.5),
                wv=weight([E, E], (2.0 / E) ** 0.5), wo=weight([E, E], (2.0 / E) ** 0.5),
                bo=const([E], 0.0), g2=const([E], 1.0), b2=const([E], 0.0),
                w1=weight([E, 4 * E], (2.0 / E) ** 0.5), bf1=const([4 * E], 0.0),
                w2=weight([4 * E, E], (0.5 / E) ** 0.5), bf2=const([E], 0.0)))
        self.gf, self.bf = const([E], 1.0), const([E], 0.0)
        self.head = weight([E, V], (2.0 / E) ** 0.5)
        # optimizer state and gradient slots
        self.m = [self.gpu(self.shape_of(p)) for p in self.params]
        self.v = [self.gpu(self.shape_of(p)) for p in self.params]
        self.grads = [None] * len(self.params)
        # inputs: embedded tokens stand-in ([T, E]) and float labels [T]
        self.x_rows = self.gpu([self.T, E])
        lab = self.cpu([self.T])
        for i, t in enumerate(seed_tokens[: self.T]):
            lib.tensor_set(lab, i, float(t))
        self.labels_host = lab            # host template; every step uploads a copy of it
        self.labels = None
        self.upload_labels()
        self.step_no = 0

    def upload_labels(self):
        """The step's labels go host -> device through the reference's own calls:
        tensor_copy (a host copy) + tensor_to_cuda (pool allocation + cudaMemcpy H2D,
        csrc/cuda/tensor.cu:17-39).  T float labels = 4 T bytes per step."""
        self.rt.cudaSetDevice(self.dev)
        if self.labels is not None:
            self.lib.tensor_free(self.labels)
        t = self.lib.tensor_copy(self.labels_host)
        self.lib.tensor_to_cuda(t)
        self.labels = t

    # -------------------------------------------------------------- helpers
    def _reg(self, t):
        self.params.append(t)
        return t

    def shape_of(self, t):
        return [t.contents.shape[i] for i in range(t.contents.ndim)]

    def _shape(self, shape):
        return (C.c_int64 * len(shape))(*shape), len(shape)

    def cpu(self, shape):
        a, n = self._shape(shape)
        return self.lib.tensor_new(a, n, 0, 0)

    def gpu(self, shape):
        a, n = self._shape(shape)
        return self.lib.tensor_new_cuda(a, n, 0)

    def view(self, t, shape):
        """Reshaped alias of `t`.  The reference's tensor_reshape bumps the source's reference
        count and its tensor_free releases the shared storage when the ALIAS is freed
        (csrc/tensor.c:108-128, 260-294), so aliases are never freed here (a few dozen bytes of
        host memory each) and the source's count is put back so it can be freed normally."""
        a, n = self._shape(shape)
        v = self.lib.tensor_reshape(t, a, n)
        t.contents.ref_count -= 1
        return v

    def free(self, *ts):
        for t in ts:
            if t:
                self.lib.tensor_free(t)

    def set_grad(self, p, g):
        i = next(k for k, q in enumerate(self.params) if C.addressof(q.contents) == C.addressof(p.contents))
        if self.grads[i]:
            self.free(self.grads[i])
        self.grads[i] = g

    def matmul_backward(self, x, w, dy, w_param):
        """dX = dY W^T, dW = X^T dY with materialised transposes, as the reference autograd does."""
        L = self.lib
        wt = L.tensor_transpose_cuda(w)
        dx = L.tensor_matmul_cuda(dy, wt)
        xt = L.tensor_transpose_cuda(x)
        dw = L.tensor_matmul_cuda(xt, dy)
        self.free(wt, xt)
        self.set_grad(w_param, dw)
        return dx

    def eltwise_standin(self, a, b, n_ops):
        """n_ops elementwise passes over tensors shaped like `a` (stand-in for a missing kernel)."""
        L = self.lib
        cur = L.tensor_mul_cuda(a, b)
        for _ in range(n_ops - 1):
            nxt = L.tensor_add_cuda(cur, b)
            self.free(cur)
            cur = nxt
        return cur

    # -------------------------------------------------------------- one step (enqueue only)
    def forward_backward(self):
        L, cfg = self.lib, self.cfg
        self.rt.cudaSetDevice(self.dev)
        E, S, Bm, H = cfg["embed"], cfg["seq"], cfg["micro_batch"], cfg["heads"]
        T, hd, BH = self.T, E // H, Bm * H
        x = L.tensor_add_cuda(self.x_rows, self.x_rows)            # embedding + positions stand-in
        saved = []
        for ly in self.layers:
            ln1 = L.tensor_fused_layernorm_cuda(x, ly["g1"], ly["b1"], 1e-5)
            q = L.tensor_matmul_cuda(ln1, ly["wq"])
            k = L.tensor_matmul_cuda(ln1, ly["wk"])
            v = L.tensor_matmul_cuda(ln1, ly["wv"])
            att = L.tensor_flash_attention_cuda(q, k, v, BH, S, hd, 1)
            o = L.tensor_matmul_cuda(att, ly["wo"])
            o2 = L.tensor_add_broadcast_cuda(o, ly["bo"])
            x1 = L.tensor_add_cuda(x, o2)
            self.free(o, o2)
            ln2 = L.tensor_fused_layernorm_cuda(x1, ly["g2"], ly["b2"], 1e-5)
            h = L.tensor_matmul_cuda(ln2, ly["w1"])
            hg = L.tensor_fused_gelu_bias_cuda(h, ly["bf1"])
            f = L.tensor_matmul_cuda(hg, ly["w2"])
            f2 = L.tensor_add_broadcast_cuda(f, ly["bf2"])
            x2 = L.tensor_add_cuda(x1, f2)
            self.free(f, f2)
            saved.append(dict(x=x, ln1=ln1, q=q, k=k, v=v, att=att, x1=x1, ln2=ln2, h=h, hg=hg))
            x = x2
        lnf = L.tensor_fused_layernorm_cuda(x, self.gf, self.bf, 1e-5)
        logits = L.tensor_matmul_cuda(lnf, self.head)
        loss = L.tensor_cross_entropy_loss_cuda(logits, self.labels)
        self.last_loss = loss
        # ---------------- backward
        dlogits = L.tensor_cross_entropy_loss_backward_cuda(logits, self.labels)
        d = self.matmul_backward(lnf, self.head, dlogits, self.head)
        self.free(dlogits, logits)
        dx = self.eltwise_standin(d, lnf, 3)                          # final LayerNorm backward
        self.set_grad(self.gf, L.tensor_add_broadcast_backward_cuda(d))
        self.set_grad(self.bf, L.tensor_add_broadcast_backward_cuda(d))
        self.free(d, lnf, x)
        for ly, sv in zip(reversed(self.layers), reversed(saved)):
            self.set_grad(ly["bf2"], L.tensor_add_broadcast_backward_cuda(dx))
            dhg = self.matmul_backward(sv["hg"], ly["w2"], dx, ly["w2"])
            dh = self.eltwise_standin(dhg, sv["h"], 3)                # GELU backward
            self.set_grad(ly["bf1"], L.tensor_add_broadcast_backward_cuda(dh))
            dln2 = self.matmul_backward(sv["ln2"], ly["w1"], dh, ly["w1"])
            t = self.eltwise_standin(dln2, sv["ln2"], 3)              # LayerNorm 2 backward
            self.set_grad(ly["g2"], L.tensor_add_broadcast_backward_cuda(dln2))
            self.set_grad(ly["b2"], L.tensor_add_broadcast_backward_cuda(dln2))
            dx1 = L.tensor_add_cuda(dx, t)
            self.free(dhg, dh, dln2, t, dx)
            self.set_grad(ly["bo"], L.tensor_add_broadcast_backward_cuda(dx1))
            datt = self.matmul_backward(sv["att"], ly["wo"], dx1, ly["wo"])
            # attention backward stand-in: 5 batched matmuls + softmax + 2 elementwise passes
            q3, k3, v3 = (self.view(sv[n], [BH, S, hd]) for n in ("q", "k", "v"))
            kT, vT = self.view(sv["k"], [BH, hd, S]), self.view(sv["v"], [BH, hd, S])
            do3 = self.view(datt, [BH, S, hd])
            sc = L.tensor_bmm_cuda(q3, kT)
            sc2 = self.view(sc, [BH * S, S])
            p2 = L.tensor_softmax_cuda(sc2)
            p3 = self.view(p2, [BH, S, S])
            dv = L.tensor_bmm_cuda(p3, do3)
            dp = L.tensor_bmm_cuda(do3, vT)
            ds = self.eltwise_standin(dp, p3, 2)
            dq = L.tensor_bmm_cuda(ds, k3)
            dk = L.tensor_bmm_cuda(ds, q3)
            self.free(sc, p2, dp, ds, datt)
            dq2, dk2, dv2 = (self.view(t_, [T, E]) for t_ in (dq, dk, dv))
            g1 = self.matmul_backward(sv["ln1"], ly["wq"], dq2, ly["wq"])
            g2 = self.matmul_backward(sv["ln1"], ly["wk"], dk2, ly["wk"])
            g3 = self.matmul_backward(sv["ln1"], ly["wv"], dv2, ly["wv"])
            s1 = L.tensor_add_cuda(g1, g2)
            dln1 = L.tensor_add_cuda(s1, g3)
            t = self.eltwise_standin(dln1, sv["ln1"], 3)              # LayerNorm 1 backward
            self.set_grad(ly["g1"], L.tensor_add_broadcast_backward_cuda(dln1))
            self.set_grad(ly["b1"], L.tensor_add_broadcast_backward_cuda(dln1))
            dx = L.tensor_add_cuda(dx1, t)
            self.free(dq, dk, dv, g1, g2, g3, s1, dln1, t, dx1)
            self.free(*(sv[n] for n in ("x", "ln1", "q", "k", "v", "att", "x1", "ln2", "h", "hg")))
        # embedding / positional scatter stand-ins: one elementwise pass each
        e1 = L.tensor_add_cuda(dx, dx)
        self.free(e1, dx)

    def grad_list(self):
        return [(i, g) for i, g in enumerate(self.grads) if g]

    def adam(self, lr, wd):
        L = self.lib
        self.rt.cudaSetDevice(self.dev)
        self.step_no += 1
        b1, b2 = 0.9, 0.95
        bc1, bc2 = 1 - b1 ** self.step_no, 1 - b2 ** self.step_no
        for i, g in self.grad_list():
            L.tensor_fused_adam_cuda(self.params[i], g, self.m[i], self.v[i], lr, b1, b2, 1e-8, bc1,
                                     bc2, wd if self.params[i].contents.ndim > 1 else 0.0)

    def read_loss(self):
        self.rt.cudaSetDevice(self.dev)
        v = self.lib.tensor_sum_cuda(self.last_loss)     # device-to-host read (synchronises)
        self.free(self.last_loss)
        return float(v)


class _ClockSampler:
    """SM clocks and throttle reasons of one GPU during the timed region (nvidia-smi, 200 ms)."""

    def __init__(self, dev=0):
        self.proc = None
        self.dev = int(dev)

    def start(self):
        import subprocess
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.dev), "--query-gpu=" + q,
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return None
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            return None
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 6 or not f[0].isdigit():
                continue
            sm.append(int(f[0]))
            mx = max(mx, int(f[1]) if f[1].isdigit() else 0)
            for nm, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        if not sm:
            return None
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm)}


def run(args, cfg):
    def emit(obj):
        obj["impl"] = "reference"
        print(json.dumps(obj), flush=True)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", str(rank)))
    if not os.path.exists(LIB_PATH):
        if rank == 0:
            emit({"unavailable": "baseline/_ref/libluatorch.so is not built (CMake build of the reference)"})
        return
    cfg = dict(cfg)
    if getattr(args, "micro_batch", 0):
        cfg["micro_batch"] = args.micro_batch
    pg = None
    if world > 1:
        # Host-side rendezvous only (barrier + max of the per-rank times).  It is imported
        # BEFORE the reference library: that library pulls in the system libnccl, and the
        # process-group package needs its own, newer one to be the first loaded.
        import torch.distributed as dist
        dist.init_process_group("gloo", rank=rank, world_size=world)
        pg = dist
    try:
        rt = C.CDLL("libcudart.so.12")
    except OSError:
        rt = C.CDLL("/usr/local/cuda/lib64/libcudart.so")
    lib = _load()
    n_dev = C.c_int(0)
    rt.cudaGetDeviceCount(C.byref(n_dev))
    # One process per GPU (the launcher starts `world` of them): each drives the unmodified
    # library on its own device.  The reference's own multi-GPU path (one process, every
    # device, luatorch_nccl_allreduce per parameter) cannot run: its single cuBLAS handle is
    # created on device 0 (csrc/cuda/ops/matmul.cu:21-35) and its one memory pool serves all
    # devices (csrc/cuda/memory_pool.cu:9-21), so a matmul on device 1 returns cuBLAS status
    # 13.  The ranks therefore exchange NO gradients: the figure is an upper bound on what
    # the reference could reach with a working exchange.
    dev = local_rank % max(1, n_dev.value)
    rt.cudaSetDevice(dev)
    lib.pool_init()
    import random
    rng = random.Random(1234 + rank)
    tokens = [rng.randrange(cfg["vocab"]) for _ in range(cfg["micro_batch"] * cfg["seq"])]
    try:
        rep = Replica(lib, rt, dev, cfg, tokens)
    except RuntimeError as e:
        if rank == 0:
            emit({"unavailable": "the reference library failed while building the model: %s" % str(e)[:200]})
        return

    def step():
        rep.upload_labels()
        rep.forward_backward()
        rep.adam(cfg["lr"], cfg["wd"])
        return rep.read_loss()

    def sync():
        rt.cudaSetDevice(dev)
        rt.cudaDeviceSynchronize()
        if pg is not None:
            pg.barrier()

    try:
        _timed_part(args, cfg, rt, lib, rep, dev, rank, world, pg, step, sync, emit)
    except RuntimeError as e:
        if rank == 0:
            emit({"unavailable": "the reference library failed on this configuration: " + str(e)[:200]})
    if pg is not None:
        pg.barrier()
        pg.destroy_process_group()
    return


def _timed_part(args, cfg, rt, lib, rep, dev, rank, world, pg, step, sync, emit):
    warmup, steps_run = max(3, args.warmup), args.steps
    for _ in range(warmup):
        step()
    sync()
    sampler = _ClockSampler(dev)
    sampler.start()
    ev0, ev1 = C.c_void_p(), C.c_void_p()
    rt.cudaSetDevice(dev)
    rt.cudaEventCreate(C.byref(ev0))
    rt.cudaEventCreate(C.byref(ev1))
    rt.cudaEventRecord(ev0, None)
    loss = None
    for _ in range(steps_run):
        loss = step()
    rt.cudaEventRecord(ev1, None)
    rt.cudaEventSynchronize(ev1)
    sync()
    ms = C.c_float(0)
    rt.cudaEventElapsedTime(C.byref(ms), ev0, ev1)
    clocks = sampler.stop()
    ms_max = ms.value
    if pg is not None:
        import torch
        t = torch.tensor([ms.value], dtype=torch.float64)
        pg.all_reduce(t, op=pg.ReduceOp.MAX)
        ms_max = float(t.item())
    if rank != 0:
        return
    B, S = cfg["micro_batch"], cfg["seq"]
    tokens_per_step = B * S * world
    value = tokens_per_step * steps_run / (ms_max * 1e-3)
    n_params = sum(int(p.contents.numel) for p in rep.params)
    note = ("ops without a reference GPU kernel are replaced by cheaper reference ops (upper bound "
            "on the reference's throughput); compute dtype fp32, the reference's only one")
    if world > 1:
        note += ("; upper bound: one process per GPU, NO gradient exchange, because the reference's "
                 "own exchange cannot run (one cuBLAS handle on device 0, csrc/cuda/ops/matmul.cu:21-35: "
                 "a matmul on device 1 returns cuBLAS status 13)")
    emit({"metric": "GPT training tokens/sec (device-timed, max over ranks)", "value": value,
          "unit": "tokens/s", "n_gpus": world, "steps": steps_run, "warmup": warmup,
          "ms_per_step": ms_max / steps_run, "higher_is_better": True, "scaling": "weak",
          "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
          "config": bench_config(getattr(args, "config", "gpt124m"), n_params, B, S, world),
          "note": note,
          "e2e": {"value": value, "unit": "tokens/s", "ms_per_step": ms_max / steps_run,
                  "h2d_bytes_per_step": 4 * B * S, "d2h_bytes_per_step": 4,
                  "note": "every timed step uploads its labels (tensor_copy + tensor_to_cuda) and "
                          "reads the loss back, so the device-timed figure is already end to end"},
          "gpu_launches": None, "clocks": clocks, "final_loss": loss})


def bench_config(name, n_params, micro_batch, seq, world):
    """The `config` block both arms of bench.py print (same keys, same values)."""
    return {"model": "GPT-%s (untied head)" % name, "global_batch": micro_batch * world,
            "micro_batch": micro_batch, "seq_len": seq, "parallelism": "dp%d" % world,
            "optimizer": "AdamW",
            "l2": "no flush: per-step working set (activations + optimizer state, > 2 GB) is far "
                  "larger than the 126 MB L2"}
