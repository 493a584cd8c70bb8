"""Headline benchmark: GPT data-parallel training tokens/sec (device-timed, max over ranks).

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...     # the unmodified reference library, same metric

Config (the reference project's GPT benchmark model scaled to the named configuration):
vocab 50257, d_model 768, 12 heads, 12 pre-LN blocks (ffn x4, GELU, causal flash attention,
dropout 0), learned positions, seq 1024, micro-batch 8 per GPU, next-token cross entropy,
AdamW lr 6e-4 wd 0.1, bf16 compute with fp32 master weights; synthetic uniform tokens,
random-init weights.  Weak scaling: per-GPU work is fixed.

The step runs through the public API; by default it is captured once into a CUDA graph
(`lf.cuda.GraphedStep`: input/target slicing, forward, loss, backward, the per-bucket fused
reduce + AdamW kernels) and replayed, `--graph 0` launches it eagerly.  Two timed regions of K
steps each, both bracketed by barrier + synchronize and timed with CUDA events on the
launching stream:
  value      steps fed from device-resident token batches (kernel-side throughput)
  e2e.value  steps through the same public API with every step's [B, S+1] tokens copied from
             pinned host memory (straight into the graph's static input) and every step's
             loss copied back to the host; the host reads each loss one step behind
             (`lf.cuda.ScalarFetcher`), so it never waits on the step it has just launched
Rank 0 prints ONE JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

CONFIGS = {
    "gpt124m": dict(vocab=50257, embed=768, heads=12, layers=12, seq=1024, micro_batch=8,
                    lr=6e-4, wd=0.1),
    "gpt1p3b": dict(vocab=50257, embed=2048, heads=16, layers=24, seq=2048, micro_batch=4,
                    lr=2e-4, wd=0.1),
    "tiny": dict(vocab=1000, embed=128, heads=2, layers=2, seq=128, micro_batch=2, lr=6e-4, wd=0.1),
}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="gpt124m", choices=sorted(CONFIGS))
    ap.add_argument("--mode", default="sharded", choices=["sharded", "replicated", "nccl"])
    ap.add_argument("--bucket-mb", type=float, default=32.0)
    ap.add_argument("--micro-batch", type=int, default=0)
    ap.add_argument("--graph", type=int, default=int(os.environ.get("LT_BENCH_GRAPH", "1")),
                    help="1 (default): replay the whole step as a CUDA graph on every rank "
                         "(lf.cuda.GraphedStep); 0: eager launches with programmatic dependent launch")
    return ap.parse_args()


def run_ours(args):
    import torch
    import torch.distributed as dist
    import luatorch_b200 as lf
    from luatorch_b200 import _C  # noqa: F401  (fail loudly without the native extension)
    from luatorch_b200.utils.timing import ClockSampler
    from baseline.reference_arm import bench_config

    cfg = dict(CONFIGS[args.config])
    if args.micro_batch:
        cfg["micro_batch"] = args.micro_batch
    warmup = max(3, args.warmup)
    lf.distributed.init()
    rank, world = lf.distributed.rank(), lf.distributed.world_size()
    dev = torch.cuda.current_device()
    lf.manual_seed(1234)
    model = lf.models.GPT(cfg["vocab"], cfg["embed"], cfg["heads"], cfg["layers"], cfg["seq"], 0.0,
                          pos="learned")
    ddp = lf.distributed.DDP(model, mode=args.mode, bucket_mb=args.bucket_mb)
    opt = lf.optim.AdamW(ddp.parameters(), cfg["lr"], 0.9, 0.95, 1e-8, cfg["wd"],
                         model.no_decay_params())
    ddp.attach(opt)
    crit = lf.nn.CrossEntropyLoss(cfg["vocab"], inplace_backward=True)
    B, S = cfg["micro_batch"], cfg["seq"]

    gen = torch.Generator().manual_seed(1000 + rank)
    n_pool = 8
    host_tokens = [torch.randint(0, cfg["vocab"], (B, S + 1), generator=gen, dtype=torch.int32).pin_memory()
                   for _ in range(n_pool)]
    dev_batches = [lf.Tensor.wrap(t.cuda()) for t in host_tokens]

    def train_step(tok):
        """One step on a [B, S+1] int32 token batch that is already on the device."""
        x = lf.Tensor.wrap(tok._t[:, :-1].contiguous())
        y = lf.Tensor.wrap(tok._t[:, 1:].contiguous().reshape(-1))
        lf.autograd.zero_graph()
        ddp.zero_grad()
        loss = crit(ddp(x), y)
        lf.autograd.backward(loss)
        ddp.sync_gradients()
        opt.step()
        return loss

    runner = None
    kernels_per_replay = 0
    if args.graph:
        # the public whole-step replay: static input tensors, one graph launch per step
        gtok = lf.Tensor.wrap(dev_batches[0]._t.clone())
        c_before = sum(lf.launch_counts())
        try:
            runner = lf.cuda.GraphedStep(lambda: train_step(gtok), opt, inputs=(gtok,), warmup=2,
                                         pdl=True)
        except Exception as e:      # capture refused on this machine: every rank goes eager
            print("bench: graph capture failed (%r), running eagerly" % (e,), file=sys.stderr)
            runner = None
        if world > 1:               # all ranks replay, or none does
            ok = torch.tensor([1 if runner is not None else 0], device="cuda")
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if int(ok.item()) == 0:
                runner = None
        # two eager warm-up steps and the capture each went through the launchers once: a
        # third of the difference is the number of this package's kernels inside the graph
        kernels_per_replay = (sum(lf.launch_counts()) - c_before) // 3 if runner is not None else 0

    def step_resident(i):
        tok = dev_batches[i % n_pool]
        return runner(tok) if runner is not None else train_step(tok)

    fetch = lf.cuda.ScalarFetcher(depth=1)
    losses = []

    def step_e2e(i):
        t = host_tokens[i % n_pool]                   # pinned host memory
        if runner is not None:
            loss = runner(t)                          # H2D straight into the graph's static input
        else:
            loss = train_step(lf.Tensor.wrap(t.to("cuda", non_blocking=True)))
        v = fetch.push(loss)                          # D2H copy of this step's loss, every step;
        if v is not None:                             # the host reads the previous step's value
            losses.append(v)
        return v

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def timed(fn, steps):
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c0 = sum(lf.launch_counts())
        e0.record()
        last = None
        for i in range(steps):
            last = fn(i)
        losses.extend(fetch.drain())      # the last steps' losses reach the host inside the region
        e1.record()
        sync_all()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, sum(lf.launch_counts()) - c0, last

    for i in range(warmup):
        step_resident(i)
    ddp.check()
    # clocks are sampled per region: the second region starts once the power limiter has settled
    # (a B200 under its 1 kW cap runs the first few hundred milliseconds of a burst faster), so
    # the two numbers differ by that as well as by the copies
    sampler = ClockSampler(dev, 0.025).start()
    ms_dev, launches, last_loss = timed(step_resident, args.steps)
    clocks = sampler.stop()
    for i in range(2):
        step_e2e(i)
    fetch.drain()
    losses.clear()
    sampler = ClockSampler(dev, 0.025).start()
    ms_e2e, _, _ = timed(step_e2e, args.steps)
    clocks_e2e = sampler.stop()
    assert len(losses) == args.steps, (len(losses), args.steps)   # one host-side loss per step
    loss_val = losses[-1]
    ddp.check()

    tokens_per_step = B * S * world
    value = tokens_per_step * args.steps / (ms_dev * 1e-3)
    e2e_value = tokens_per_step * args.steps / (ms_e2e * 1e-3)
    if rank == 0:
        out = {
            "metric": "GPT training tokens/sec (device-timed, max over ranks)",
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": ms_dev / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "impl": "ours",
            # the same keys and values as the reference arm prints (baseline/reference_arm.py)
            "config": bench_config(args.config, model.num_params(), B, S, world),
            "engine": {"params": model.num_params(), "dp_mode": ddp.mode, "nvls": bool(ddp.nvls),
                       "state_sharded": ddp.arena.state_shards is not None,
                       "buckets": len(ddp.buckets), "cuda_graph": runner is not None,
                       # fp32 master + two moments held by THIS rank, and the allocator's peak
                       "optimizer_state_gb": round(3 * 4 * ddp.arena.state_numel() / 1e9, 3),
                       "peak_memory_gb": round(torch.cuda.max_memory_allocated() / 1e9, 2)},
            "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": B * (S + 1) * 4, "d2h_bytes_per_step": 4,
                    "final_loss": loss_val, "clocks": clocks_e2e},
            # host launches counted in the timed region, plus the kernels each graph replay runs
            "gpu_launches": int(launches + kernels_per_replay * args.steps),
            "clocks": clocks,
        }
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
    lf.distributed.destroy()


def run_reference(args):
    try:
        from baseline.reference_arm import run as ref_run
    except Exception as e:  # the arm lives beside the reference install
        print(json.dumps({"impl": "reference", "unavailable": "reference arm not importable: %r" % (e,)}))
        return
    ref_run(args, CONFIGS[args.config])


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
