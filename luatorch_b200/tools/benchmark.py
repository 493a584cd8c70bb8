"""Kernel micro-benchmarks with a roofline column (counterpart of the reference's
tools/benchmark.lua, which times ops with os.clock() and no device synchronise, :14-27).

    python -m luatorch_b200.tools.benchmark                 # the whole table
    python -m luatorch_b200.tools.benchmark --only gemm --iters 3 --warmup 1   # small, for ncu
    python -m luatorch_b200.tools.benchmark --csv out.csv

Every row is timed with CUDA events on the launching stream after warm-up, with a synchronise
on both sides; between iterations a buffer larger than L2 is rewritten unless the operands
themselves exceed L2.  Fractions are relative to the measured peaks in MEASURED_PEAKS.json at
the repository root when that file exists (copy bandwidth and cuBLAS bf16 throughput of the
same machine), else to 6.65 TB/s and 1.59 PFLOP/s.
"""
from __future__ import annotations

import argparse
import json
import math
import os

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"] * 1e9, d["bf16_tflops"] * 1e12, "measured"
    return 6.65e12, 1.59e15, "fallback"


class Timer:
    def __init__(self, iters, warmup, flush=True):
        self.iters, self.warmup = iters, warmup
        self.flush_buf = torch.empty(192 * 1024 * 1024, dtype=torch.uint8, device="cuda") if flush else None

    def __call__(self, fn, big_operands=False):
        for _ in range(self.warmup):
            fn()
        torch.cuda.synchronize()
        total = 0.0
        for _ in range(self.iters):
            if self.flush_buf is not None and not big_operands:
                self.flush_buf.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        return total / self.iters


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="", help="comma list of: gemm,gemm_epilogue,attention,layernorm,softmax_ce,elementwise,adamw,embedding")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--csv", default="")
    ap.add_argument("--shape", default="", help="gemm only: M,N,K override")
    ap.add_argument("--adamw-params", type=int, default=163_000_064,
                    help="adamw only: parameter count (a smaller one keeps an ncu capture short)")
    args = ap.parse_args(argv)
    from luatorch_b200 import _backend as B
    C = B.ext()
    hbm, tc, src = peaks()
    only = set(filter(None, args.only.split(",")))
    timer = Timer(args.iters, args.warmup)
    rows = []

    def add(group, name, ms, flops=0.0, bytes_=0.0):
        frac = max(flops / tc, bytes_ / hbm) / (ms * 1e-3) if ms > 0 else 0.0
        rows.append((group, name, ms, flops / ms / 1e9 if flops else 0.0, bytes_ / ms / 1e6 if bytes_ else 0.0, frac))
        print("%-11s %-44s %9.4f ms %9.1f TFLOP/s %9.1f GB/s  %5.1f%% of %s roofline" % (
            group, name, ms, rows[-1][3], rows[-1][4], 100 * frac, src), flush=True)

    bf = torch.bfloat16
    if not only or "gemm" in only:
        shapes = [(8192, 2304, 768, False, True), (8192, 768, 768, False, True), (8192, 3072, 768, False, True),
                  (8192, 768, 3072, False, True), (8192, 768, 3072, False, False), (768, 3072, 8192, True, True),
                  (8192, 50257, 768, False, True), (8192, 8192, 8192, False, True), (8192, 8192, 2048, False, True)]
        if args.shape:
            m, n, k = (int(v) for v in args.shape.split(","))
            shapes = [(m, n, k, False, True)]
        for M, N, K, a_t, b_n in shapes:
            a = (torch.randn((K, M) if a_t else (M, K), device="cuda") * 0.1).to(bf)
            ldb = (N + 7) // 8 * 8
            b = (torch.randn((K, ldb) if b_n else (N, K), device="cuda") * 0.1).to(bf)
            out = torch.empty((M, ldb), device="cuda", dtype=bf)[:, :N]
            ms = timer(lambda: B.gemm(a, b, a_t=a_t, b_t=not b_n, out=out, n_valid=N),
                       big_operands=(M * K + K * N + M * N) * 2 > 150e6)
            add("gemm", "bf16 [%d,%d]x[%d,%d] %s%s" % (M, K, K, N, "At" if a_t else "A", "B" if b_n else "Bt"), ms,
                2.0 * M * N * K, 2.0 * (M * K + K * N + M * N))
    if not only or "gemm_epilogue" in only:
        # the fused epilogues of one GPT-124M MLP block against the plain product of the same shape
        M, K, N = 8192, 768, 3072
        x = (torch.randn(M, K, device="cuda") * 0.1).to(bf)
        w1 = (torch.randn(K, N, device="cuda") * 0.05).to(bf)
        w2 = (torch.randn(N, K, device="cuda") * 0.05).to(bf)
        bias = torch.randn(N, device="cuda").to(bf)
        out = torch.empty(M, N, device="cuda", dtype=bf)
        pre = torch.empty_like(out)
        res = torch.randn(M, K, device="cuda").to(bf)
        out_k = torch.empty(M, K, device="cuda", dtype=bf)
        fl = 2.0 * M * N * K
        nb_ops = 2.0 * (M * K + K * N)
        nb_out = 2.0 * M * N
        for name, fn, nbytes in [
            ("[8192,768]x[768,3072] plain", lambda: B.gemm(x, w1, out=out), nb_ops + nb_out),
            ("  + bias", lambda: B.gemm(x, w1, bias=bias, out=out), nb_ops + nb_out),
            ("  + bias + GELU + pre-activation out", lambda: B.gemm(x, w1, bias=bias, act=1, aux_out=pre, out=out), nb_ops + 2 * nb_out),
            ("[8192,768]x[3072,768]^T plain (dgrad)", lambda: B.gemm(x, w2, b_t=True, out=out), nb_ops + nb_out),
            ("  * GELU'(pre-activation in)", lambda: B.gemm(x, w2, b_t=True, act=2, aux_in=pre, out=out), nb_ops + 2 * nb_out),
            ("[8192,3072]x[3072,768] plain", lambda: B.gemm(out, w2, out=out_k), 2.0 * (M * N + N * K + M * K)),
            ("  + bias + residual", lambda: B.gemm(out, w2, bias=bias[:K].contiguous(), residual=res, out=out_k),
             2.0 * (M * N + N * K + 2 * M * K)),
        ]:
            add("gemm_epi", name, timer(fn), fl, nbytes)
    if not only or "attention" in only:
        for Bn, S, H, D in [(8, 1024, 12, 64), (4, 2048, 16, 128)]:
            qkv = (torch.randn(Bn, S, 3, H, D, device="cuda") * 0.5).to(bf)
            q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
            sc = 1.0 / math.sqrt(D)
            o, lse = C.flash_forward(q, k, v, True, sc)
            d_o = torch.randn_like(o)
            fl = 4.0 * Bn * H * S * S * D / 2
            add("attention", "flash fwd causal B%d S%d H%d D%d" % (Bn, S, H, D),
                timer(lambda: C.flash_forward(q, k, v, True, sc)), fl, 8.0 * Bn * S * H * D)
            add("attention", "flash bwd causal B%d S%d H%d D%d" % (Bn, S, H, D),
                timer(lambda: C.flash_backward(q, k, v, o, lse, d_o, True, sc, None)), 2.5 * fl, 16.0 * Bn * S * H * D)
    if not only or "layernorm" in only:
        for rows_, cols in [(8192, 768), (8192, 2048)]:
            x = torch.randn(rows_, cols, device="cuda").to(bf)
            g = torch.ones(cols, device="cuda", dtype=bf)
            y, mean, rstd = C.layernorm_forward(x, g, g, 1e-5)
            dg = torch.zeros(cols, device="cuda")
            db = torch.zeros(cols, device="cuda")
            nb = rows_ * cols * 2
            add("layernorm", "fwd [%d,%d] bf16" % (rows_, cols), timer(lambda: C.layernorm_forward(x, g, g, 1e-5)), 0, 2 * nb)
            add("layernorm", "bwd [%d,%d] bf16" % (rows_, cols),
                timer(lambda: C.layernorm_backward(x, y, g, mean, rstd, None, dg, db, False)), 0, 3 * nb)
    if not only or "softmax_ce" in only:
        rows_, cols, ld = 8192, 50257, 50264
        logits = torch.randn(rows_, ld, device="cuda").to(bf)[:, :cols]
        labels = torch.randint(0, cols, (rows_,), device="cuda")
        loss, lse, err = C.cross_entropy_forward(logits, cols, labels)
        nb = rows_ * cols * 2
        add("softmax_ce", "CE fwd [%d,%d] bf16" % (rows_, cols), timer(lambda: C.cross_entropy_forward(logits, cols, labels), True), 0, nb)
        add("softmax_ce", "CE bwd in place [%d,%d] bf16" % (rows_, cols),
            timer(lambda: C.cross_entropy_backward(logits, cols, labels, lse, 1.0 / rows_, None, logits), True), 0, 2 * nb)
        logits2 = torch.randn(rows_, ld, device="cuda").to(bf)
        add("softmax_ce", "CE fused fwd+bwd in place [%d,%d] bf16" % (rows_, cols),
            timer(lambda: C.cross_entropy_fused(logits2, cols, labels, 1.0 / rows_), True), 0, 2 * nb)
    if not only or "elementwise" in only:
        n = 1 << 28
        a = torch.randn(n, device="cuda").to(bf)
        b = torch.randn(n, device="cuda").to(bf)
        add("elementwise", "add bf16 2^28", timer(lambda: C.binary(0, a, b, False), True), 0, 3 * n * 2)
        add("elementwise", "gelu bf16 2^28", timer(lambda: C.unary(8, a), True), 0, 2 * n * 2)
        add("elementwise", "sum bf16 2^28", timer(lambda: C.reduce(0, a, 1.0), True), 0, n * 2)
    if not only or "adamw" in only:
        n = args.adamw_params // 8 * 8
        master = torch.randn(n, device="cuda")
        shadow = torch.empty(n, device="cuda", dtype=bf)
        grad = torch.randn(n, device="cuda").to(bf)
        m = torch.zeros(n, device="cuda")
        v = torch.zeros(n, device="cuda")
        add("adamw", "flat AdamW %dM params (bf16 grad, bf16 shadow)" % (n // 1_000_000),
            timer(lambda: C.adamw_flat(master, shadow, grad, m, v, None, None, 1e-3, 0.9, 0.95, 1e-8, 0.1, 0.05, 1.0, None), True),
            0, n * 28.0)
    if not only or "embedding" in only:
        vocab, dim, T = 50257, 768, 8192
        table = torch.randn(vocab, dim, device="cuda").to(bf)
        ids = torch.randint(0, vocab, (T,), device="cuda")
        dy = torch.randn(T, dim, device="cuda").to(bf)
        dt = torch.empty(vocab, dim, device="cuda", dtype=bf)
        add("embedding", "gather 8192 x 768", timer(lambda: C.embedding_forward(table, ids, None, 1)), 0, 2 * T * dim * 2)
        add("embedding", "scatter-add into [50257,768]", timer(lambda: C.embedding_backward(dy, ids, dt, False)), 0,
            (T + vocab) * dim * 2)
    if args.csv:
        with open(args.csv, "w") as f:
            f.write("group,name,ms,tflops,gbs,roofline_fraction\n")
            for r in rows:
                f.write("%s,%s,%.5f,%.2f,%.1f,%.4f\n" % r)


if __name__ == "__main__":
    main()
