"""XOR on the CPU in fp32 (examples/xor.lua, test/test_training.lua:11-50):
Linear(2,8)-Tanh-Linear(8,1)-Sigmoid, MSE, Adam lr 0.01, 2000 full-batch steps, seeded
weights, then a checkpoint round trip."""
from __future__ import annotations

import argparse
import os
import tempfile

import luatorch_b200 as lf


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--hidden", type=int, default=8)
    ap.add_argument("--lr", type=float, default=0.01)
    ap.add_argument("--seed", type=int, default=1234)
    args = ap.parse_args(argv)
    lf.manual_seed(args.seed)
    nn = lf.nn
    model = nn.Sequential(nn.Linear(2, args.hidden), nn.Tanh(), nn.Linear(args.hidden, 1), nn.Sigmoid())
    crit = nn.MSELoss()
    opt = lf.optim.Adam(model.parameters(), args.lr)
    x = lf.Tensor.from_list([0, 0, 0, 1, 1, 0, 1, 1], [4, 2])
    y = lf.Tensor.from_list([0, 1, 1, 0], [4, 1])
    logger = lf.utils.Logger(max(1, args.steps // 10))
    for _ in range(args.steps):
        lf.autograd.zero_graph()
        model.zero_grad()
        loss = crit(model(x), y)
        lf.autograd.backward(loss)
        opt.step()
        logger.log(loss.get(0), None, opt.lr)
    pred = model(x)
    for i in range(4):
        print("%d xor %d -> %.4f" % (x.get(2 * i), x.get(2 * i + 1), pred.get(i)))
    path = os.path.join(tempfile.gettempdir(), "luatorch_b200_xor.bin")
    lf.io.checkpoint.save(model, path)
    fresh = nn.Sequential(nn.Linear(2, args.hidden), nn.Tanh(), nn.Linear(args.hidden, 1), nn.Sigmoid())
    lf.io.checkpoint.load(fresh, path)
    diff = max(abs(fresh(x).get(i) - pred.get(i)) for i in range(4))
    print("final loss %.5f, checkpoint round-trip max diff %.2e" % (loss.get(0), diff))
    return loss.get(0)


if __name__ == "__main__":
    main()
