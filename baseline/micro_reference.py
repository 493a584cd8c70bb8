"""Per-op micro-baselines of the UNMODIFIED reference library (baseline/_ref/libluatorch.so,
built from the reference sources with CMake), called through its C ABI at the shapes of the
GPT-124M configuration.  One line per op: device time (CUDA events on the default stream the
reference launches on, after warm-up, a synchronise on both sides) and the derived rate.

    python -m baseline.micro_reference [--iters 5] [--csv out.csv]

Ops timed (reference entry point, file:line of the kernel behind it):
  tensor_matmul_cuda            cuBLAS SGEMM            csrc/cuda/ops/matmul.cu:92-141
  tensor_flash_attention_cuda   forward only            csrc/cuda/ops/flash_attention.cu:19-145
  tensor_fused_layernorm_cuda   forward only            csrc/cuda/ops/fused.cu:63-127
  tensor_fused_gelu_bias_cuda                           csrc/cuda/ops/fused.cu:26-58
  tensor_cross_entropy_loss[_backward]_cuda             csrc/cuda/ops/loss.cu:63-125
  tensor_fused_adam_cuda        one launch per tensor   csrc/cuda/ops/fused.cu:132-174
  tensor_sum_cuda               host-finished reduce    csrc/cuda/ops/arithmetic.cu:339-380
  tensor_add_cuda                                       csrc/cuda/ops/arithmetic.cu:57-60
Every out-of-place reference op allocates and zero-fills its output inside the call
(csrc/cuda/tensor.cu:70-113); that cost is part of the op as a user of the reference pays it.
"""
from __future__ import annotations

import argparse
import ctypes as C
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from baseline.reference_arm import LIB_PATH, TP, _load  # noqa: E402


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--csv", default="")
    args = ap.parse_args(argv)
    if not os.path.exists(LIB_PATH):
        print("unavailable: baseline/_ref/libluatorch.so is not built")
        return 0
    try:
        rt = C.CDLL("libcudart.so.12")
    except OSError:
        rt = C.CDLL("/usr/local/cuda/lib64/libcudart.so")
    lib = _load()
    lib.tensor_free.argtypes = [TP]
    rt.cudaSetDevice(0)
    lib.pool_init()

    def gpu(shape, fill=None, randn=False):
        a = (C.c_int64 * len(shape))(*shape)
        if fill is None and not randn:
            return lib.tensor_new_cuda(a, len(shape), 0)
        t = lib.tensor_new(a, len(shape), 0, 0)
        if randn:
            lib.tensor_randn(t)
        else:
            lib.tensor_fill(t, fill)
        lib.tensor_to_cuda(t)
        return t

    ev0, ev1 = C.c_void_p(), C.c_void_p()
    rt.cudaEventCreate(C.byref(ev0))
    rt.cudaEventCreate(C.byref(ev1))
    flush = gpu([64 * 1024 * 1024])       # 256 MB fp32, rewritten between iterations

    def timed(fn):
        for _ in range(args.warmup):
            r = fn()
            if r:
                lib.tensor_free(r)
        total = 0.0
        for _ in range(args.iters):
            lib.tensor_mul_scalar_cuda_(flush, 1.0)       # evicts L2
            rt.cudaDeviceSynchronize()
            rt.cudaEventRecord(ev0, None)
            r = fn()
            rt.cudaEventRecord(ev1, None)
            rt.cudaEventSynchronize(ev1)
            ms = C.c_float(0)
            rt.cudaEventElapsedTime(C.byref(ms), ev0, ev1)
            total += ms.value
            if r:
                lib.tensor_free(r)
        return total / args.iters

    rows = []

    def report(name, ms, flops=0.0, nbytes=0.0):
        rows.append((name, ms, flops / ms / 1e9 if flops else 0.0, nbytes / ms / 1e6 if nbytes else 0.0))
        print("%-58s %10.4f ms %9.1f TFLOP/s %9.1f GB/s" % rows[-1], flush=True)

    M = 8192
    for K, N in ((768, 768), (768, 2304), (768, 3072), (3072, 768), (768, 50257)):
        a, b = gpu([M, K], randn=True), gpu([K, N], randn=True)
        ms = timed(lambda: lib.tensor_matmul_cuda(a, b))
        report("tensor_matmul_cuda fp32 [%d,%d]x[%d,%d]" % (M, K, K, N), ms, 2.0 * M * N * K,
               4.0 * (M * K + K * N + M * N))
        lib.tensor_free(a)
        lib.tensor_free(b)

    BH, S, D = 96, 1024, 64
    q, k, v = (gpu([BH, S, D], randn=True) for _ in range(3))
    ms = timed(lambda: lib.tensor_flash_attention_cuda(q, k, v, BH, S, D, 1))
    report("tensor_flash_attention_cuda causal (96,1024,64) fwd", ms, 4.0 * BH * S * S * D / 2)
    for t in (q, k, v):
        lib.tensor_free(t)

    x, g, b = gpu([M, 768], randn=True), gpu([768], fill=1.0), gpu([768], fill=0.0)
    ms = timed(lambda: lib.tensor_fused_layernorm_cuda(x, g, b, 1e-5))
    report("tensor_fused_layernorm_cuda [8192,768] fwd", ms, 0, 8.0 * M * 768)
    for t in (x, g, b):
        lib.tensor_free(t)

    x, b = gpu([M, 3072], randn=True), gpu([3072], fill=0.1)
    ms = timed(lambda: lib.tensor_fused_gelu_bias_cuda(x, b))
    report("tensor_fused_gelu_bias_cuda [8192,3072]", ms, 0, 8.0 * M * 3072)
    ms = timed(lambda: lib.tensor_add_cuda(x, x))
    report("tensor_add_cuda [8192,3072]", ms, 0, 12.0 * M * 3072)
    ms = timed(lambda: (lib.tensor_sum_cuda(x), None)[1])
    report("tensor_sum_cuda [8192,3072] (host-finished)", ms, 0, 4.0 * M * 3072)
    lib.tensor_free(x)
    lib.tensor_free(b)

    V = 50257
    logits, labels = gpu([M, V], randn=True), gpu([M], fill=7.0)
    ms = timed(lambda: lib.tensor_cross_entropy_loss_cuda(logits, labels))
    report("tensor_cross_entropy_loss_cuda [8192,50257]", ms, 0, 4.0 * M * V)
    ms = timed(lambda: lib.tensor_cross_entropy_loss_backward_cuda(logits, labels))
    report("tensor_cross_entropy_loss_backward_cuda [8192,50257]", ms, 0, 8.0 * M * V)
    lib.tensor_free(logits)
    lib.tensor_free(labels)

    # AdamW over the GPT-124M parameter list: one launch per tensor, as the optimizer does
    E, L = 768, 12
    shapes = [[V, E], [1024, E]]
    for _ in range(L):
        shapes += [[E], [E], [E, E], [E, E], [E, E], [E, E], [E], [E], [E], [E, 4 * E], [4 * E],
                   [4 * E, E], [E]]
    shapes += [[E], [E], [E, V]]
    ps = [(gpu(s, fill=0.01), gpu(s, fill=0.001), gpu(s), gpu(s)) for s in shapes]
    n_par = sum(p[0].contents.numel for p in ps)

    def adam_all():
        for p, g_, m_, v_ in ps:
            lib.tensor_fused_adam_cuda(p, g_, m_, v_, 6e-4, 0.9, 0.999, 1e-8, 0.1, 0.001, 0.1)
        return None

    ms = timed(adam_all)
    report("tensor_fused_adam_cuda x%d tensors (%.0fM params)" % (len(ps), n_par / 1e6), ms, 0,
           28.0 * n_par)

    if args.csv:
        with open(args.csv, "w") as f:
            f.write("name,ms,tflops,gbs\n")
            for r in rows:
                f.write("%s,%.5f,%.2f,%.1f\n" % r)
    return 0


if __name__ == "__main__":
    sys.exit(main())
