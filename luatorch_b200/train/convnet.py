"""Conv net, data parallel: synthetic images [batch 128 per GPU, 3, 32, 32] ~ N(0,1), labels
uniform in [0,10); Conv2d(3,32,3,1,1)-ReLU-Conv2d(32,64,3,2,1)-ReLU-Conv2d(64,128,3,2,1)-ReLU-
flatten-Linear(8192,10), cross entropy, SGD momentum 0.9, bf16.  (The reference's
examples/cifar.lua falls back to an MLP because its convolution runs im2col on the CPU and has
no input gradient.)"""
from __future__ import annotations

import argparse

import torch

import luatorch_b200 as lf
from .common import StepTimer, log, max_over_ranks


class ConvNet(lf.nn.Module):
    def __init__(self):
        nn = lf.nn
        self.c1, self.c2, self.c3 = nn.Conv2d(3, 32, 3, 1, 1), nn.Conv2d(32, 64, 3, 2, 1), nn.Conv2d(64, 128, 3, 2, 1)
        self.fc = nn.Linear(8192, 10, pad_out=True)   # row stride 16: TMA-addressable, tensor-core path

    def children(self):
        return [self.c1, self.c2, self.c3, self.fc]

    def parameters(self):
        return self.c1.parameters() + self.c2.parameters() + self.c3.parameters() + self.fc.parameters()

    def forward(self, x, batch):
        nn, ag = lf.nn, lf.autograd
        h, oh, ow = self.c1(x, batch, 32, 32, act="relu")
        h = nn.to_nchw(h, batch, 32, oh * ow)
        h, oh, ow = self.c2(h, batch, oh, ow, act="relu")
        h = nn.to_nchw(h, batch, 64, oh * ow)
        h, oh, ow = self.c3(h, batch, oh, ow, act="relu")
        h = nn.to_nchw(h, batch, 128, oh * ow)
        flat = lf.Tensor.wrap(h._t.reshape(batch, 8192))
        ag.record("flatten", [h], flat, lambda g: ag.acc_grad(h, g._t.reshape(h._t.shape)))
        return self.fc(flat)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--batch", type=int, default=128)
    ap.add_argument("--mode", default="auto", choices=["auto", "replicated", "sharded", "nccl"])
    ap.add_argument("--graph", action="store_true", help="replay the step as a CUDA graph (every rank replays its own capture)")
    args = ap.parse_args(argv)
    lf.distributed.init()
    rank, world = lf.distributed.rank(), lf.distributed.world_size()
    lf.manual_seed(2)
    model = ConvNet()
    cuda = torch.cuda.is_available()
    dev = "cuda" if cuda else "cpu"
    ddp = lf.distributed.DDP(model, mode=args.mode, device=dev)
    opt = lf.optim.SGD(ddp.parameters(), 0.01, 0.9)
    ddp.attach(opt)
    crit = lf.nn.CrossEntropyLoss()
    g = torch.Generator().manual_seed(200 + rank)
    x = lf.Tensor.wrap(torch.randn(args.batch * 3 * 32 * 32, generator=g).to(dev))
    y = lf.Tensor.wrap(torch.randint(0, 10, (args.batch,), generator=g).float().to(dev))

    def one_step():
        lf.autograd.zero_graph()
        ddp.zero_grad()
        loss = crit(model.forward(x, args.batch), y)
        lf.autograd.backward(loss)
        ddp.sync_gradients()
        opt.step()
        return loss

    if args.graph and cuda:
        one_step = lf.cuda.GraphedStep(one_step, opt, inputs=(x, y))
    timer = StepTimer()
    for step in range(args.steps):
        loss = one_step()
        if rank == 0 and (step + 1) % max(1, args.steps // 5) == 0:
            print("step %5d  loss %.4f" % (step + 1, loss.item()), flush=True)
    ms = max_over_ranks(timer.elapsed_ms())
    ddp.check()
    log("convnet: %d steps, %.3f ms/step, %.0f images/s over %d gpu(s)" % (
        args.steps, ms / args.steps, args.batch * world * args.steps / (ms * 1e-3), world))
    lf.distributed.destroy()


if __name__ == "__main__":
    main()
