"""Per-step latency of the tiny XOR network (examples/benchmark_pytorch.lua:1-150): the
2-16-1 Tanh/Sigmoid model, MSE, Adam lr 0.05, 1000 full-batch steps.  Reports total time,
mean / p50 / p95 / p99 / max per step, steps per second, host and device memory, the four
predictions, and optionally a CSV of the per-step times - and, because the point of that
script is a comparison with PyTorch, runs the same network on stock torch.nn beside it.

    python -m luatorch_b200.tools.xor_benchmark [--device cpu|cuda] [--graph] [--csv out.csv]

Host time per step is measured with perf_counter (the step ends with a read of the loss, as in
the reference's loop, so on CUDA it includes the device work).  `--graph` (CUDA) replays the
step as one CUDA graph.
"""
from __future__ import annotations

import argparse
import resource
import sys
import time

import torch

import luatorch_b200 as lf

XOR_X = [0, 0, 0, 1, 1, 0, 1, 1]
XOR_Y = [0, 1, 1, 0]


def percentile(values, p: float) -> float:
    """Nearest-rank percentile, p in (0, 1]."""
    s = sorted(values)
    idx = min(len(s), max(1, -(-len(s) * p // 1)))
    return s[int(idx) - 1]


def summarize(name: str, times_ms, final_loss: float, out=sys.stdout) -> dict:
    total = sum(times_ms) / 1e3
    stats = {"name": name, "steps": len(times_ms), "final_loss": final_loss, "total_s": total,
             "avg_ms": sum(times_ms) / len(times_ms), "p50_ms": percentile(times_ms, 0.50),
             "p95_ms": percentile(times_ms, 0.95), "p99_ms": percentile(times_ms, 0.99),
             "max_ms": max(times_ms), "steps_per_s": len(times_ms) / total if total else 0.0}
    print("%s\n%s" % (name, "-" * 40), file=out)
    print("steps:               %d" % stats["steps"], file=out)
    print("final loss:          %.6f" % final_loss, file=out)
    print("total time:          %.3f sec" % total, file=out)
    for key, label in (("avg_ms", "avg time per step: "), ("p50_ms", "median per step:   "),
                       ("p95_ms", "p95 per step:      "), ("p99_ms", "p99 per step:      "),
                       ("max_ms", "max per step:      ")):
        print("%s  %.3f ms" % (label, stats[key]), file=out)
    print("steps/sec:           %.0f" % stats["steps_per_s"], file=out)
    return stats


def run_framework(steps: int, device: str, graph: bool, seed: int):
    lf.manual_seed(seed)
    nn = lf.nn
    model = nn.Sequential(nn.Linear(2, 16), nn.Tanh(), nn.Linear(16, 1), nn.Sigmoid())
    x = lf.Tensor.from_list(XOR_X, [4, 2])
    y = lf.Tensor.from_list(XOR_Y, [4, 1])
    arena = None
    if device == "cuda":
        arena = lf.cuda.amp.autocast_bf16(model)       # parameters into a flat arena on the GPU
        x, y = x.cuda(), y.cuda()
    opt = lf.optim.Adam(model.parameters(), 0.05)
    crit = nn.MSELoss()

    def one_step():
        lf.autograd.zero_graph()
        if arena is not None:
            arena.zero_grad()
        else:
            model.zero_grad()
        loss = crit(model(x), y)
        lf.autograd.backward(loss)
        opt.step()
        return loss

    if graph and device == "cuda":
        one_step = lf.cuda.GraphedStep(one_step, opt, inputs=(x, y))
    times, final = [], 0.0
    for _ in range(steps):
        t0 = time.perf_counter()
        final = one_step().get(0)
        times.append((time.perf_counter() - t0) * 1e3)
    with lf.autograd.no_grad():
        pred = model(x)
        preds = [pred.get(i) for i in range(4)]
    return model, times, final, preds


def run_torch(steps: int, device: str, seed: int):
    torch.manual_seed(seed)
    tnn = torch.nn
    model = tnn.Sequential(tnn.Linear(2, 16), tnn.Tanh(), tnn.Linear(16, 1), tnn.Sigmoid()).to(device)
    x = torch.tensor(XOR_X, dtype=torch.float32, device=device).reshape(4, 2)
    y = torch.tensor(XOR_Y, dtype=torch.float32, device=device).reshape(4, 1)
    opt = torch.optim.Adam(model.parameters(), lr=0.05)
    times, final = [], 0.0
    for _ in range(steps):
        t0 = time.perf_counter()
        opt.zero_grad(set_to_none=True)
        loss = torch.nn.functional.mse_loss(model(x), y)
        loss.backward()
        opt.step()
        final = loss.item()
        times.append((time.perf_counter() - t0) * 1e3)
    with torch.no_grad():
        preds = model(x).reshape(-1).tolist()
    return times, final, preds


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--device", default="cpu", choices=["cpu", "cuda"])
    ap.add_argument("--graph", action="store_true", help="CUDA only: replay the step as a CUDA graph")
    ap.add_argument("--seed", type=int, default=1234)
    ap.add_argument("--csv", default="", help="write per-step times (ms) of both arms to this file")
    ap.add_argument("--no-torch", action="store_true", help="skip the stock PyTorch arm")
    args = ap.parse_args(argv)
    if args.device == "cuda" and not torch.cuda.is_available():
        print("cuda requested but no GPU is visible; running on the cpu")
        args.device = "cpu"
    rss0 = resource.getrusage(resource.RUSAGE_SELF).ru_maxrss
    model, times, final, preds = run_framework(args.steps, args.device, args.graph, args.seed)
    rss1 = resource.getrusage(resource.RUSAGE_SELF).ru_maxrss
    print("luatorch_b200 XOR benchmark (%s%s)" % (args.device, ", graph replay" if args.graph else ""))
    print("model: %r" % model)
    print("parameters: %d\n" % model.num_params())
    ours = summarize("luatorch_b200", times, final)
    print("host memory peak:    %.1f MB (+%.1f MB during training)" % (rss1 / 1024, (rss1 - rss0) / 1024))
    if args.device == "cuda":
        print("gpu memory:          %.1f MB" % (lf.Tensor.cuda_memory_allocated() / 2**20))
    print("\npredictions:")
    for i in range(4):
        print("  %d xor %d = %.4f (target: %d)" % (XOR_X[2 * i], XOR_X[2 * i + 1], preds[i], XOR_Y[i]))
    theirs, t_times = None, []
    if not args.no_torch:
        t_times, t_final, t_preds = run_torch(args.steps, args.device, args.seed)
        print()
        theirs = summarize("stock torch.nn (same network, same optimizer)", t_times, t_final)
        print("\nmedian step: luatorch_b200 %.3f ms vs torch %.3f ms (%.2fx)" % (
            ours["p50_ms"], theirs["p50_ms"], theirs["p50_ms"] / ours["p50_ms"] if ours["p50_ms"] else 0.0))
    if args.csv:
        with open(args.csv, "w") as f:
            f.write("step,time_ms,torch_time_ms\n")
            for i, t in enumerate(times):
                f.write("%d,%.4f,%s\n" % (i + 1, t, "%.4f" % t_times[i] if i < len(t_times) else ""))
        print("\nper-step timings saved to %s" % args.csv)
    return ours, theirs


if __name__ == "__main__":
    main()
