"""MLP classifier, data parallel (the reference's README quick start / examples/mnist.lua):
synthetic inputs [batch 256, 784] uniform in [0,1], labels uniform in [0,10),
Linear(784,256)-ReLU-Dropout(0.2)-Linear(256,10), cross entropy, Adam lr 1e-3, bf16 compute
with fp32 master weights.  With more than one rank the whole model is one small gradient
bucket, so this exercises the one-shot fused all-reduce + Adam kernel.  `--graph` replays the
whole step as a CUDA graph on every rank (the step is launch-bound)."""
from __future__ import annotations

import argparse

import torch

import luatorch_b200 as lf
from .common import StepTimer, log, max_over_ranks


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--mode", default="auto", choices=["auto", "replicated", "sharded", "nccl"])
    ap.add_argument("--graph", action="store_true", help="replay the step as a CUDA graph (every rank replays its own capture)")
    args = ap.parse_args(argv)
    lf.distributed.init()
    rank, world = lf.distributed.rank(), lf.distributed.world_size()
    lf.manual_seed(1)
    nn = lf.nn
    model = nn.Sequential(nn.Linear(784, 256), nn.ReLU(), nn.Dropout(0.2), nn.Linear(256, 10))
    cuda = torch.cuda.is_available()
    ddp = lf.distributed.DDP(model, mode=args.mode, device="cuda" if cuda else "cpu")
    opt = lf.optim.Adam(ddp.parameters(), 1e-3)
    ddp.attach(opt)
    crit = nn.CrossEntropyLoss()
    g = torch.Generator().manual_seed(100 + rank)
    dev = "cuda" if cuda else "cpu"
    x = lf.Tensor.wrap(torch.rand(args.batch, 784, generator=g).to(dev))
    y = lf.Tensor.wrap(torch.randint(0, 10, (args.batch,), generator=g).float().to(dev))
    logger = lf.utils.Logger(max(1, args.steps // 5))

    def one_step():
        lf.autograd.zero_graph()
        ddp.zero_grad()
        loss = crit(ddp(x), y)
        lf.autograd.backward(loss)
        ddp.sync_gradients()
        opt.step()
        return loss

    if args.graph and cuda:
        one_step = lf.cuda.GraphedStep(one_step, opt, inputs=(x, y))
    timer = StepTimer()
    for step in range(args.steps):
        loss = one_step()
        if (step + 1) % logger.print_every == 0 and rank == 0:
            logger.step = step
            logger.log(loss.item(), None, opt.lr)
    ms = max_over_ranks(timer.elapsed_ms())
    ddp.check()
    log("mlp: %d steps, %.3f ms/step, %.0f samples/s over %d gpu(s), final loss %.4f" % (
        args.steps, ms / args.steps, args.batch * world * args.steps / (ms * 1e-3), world, loss.item()))
    lf.distributed.destroy()


if __name__ == "__main__":
    main()
