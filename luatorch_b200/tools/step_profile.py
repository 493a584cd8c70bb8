"""Per-kernel breakdown of a GPT training step, measured in place (kernels keep the cache and
clock state the step gives them, unlike a kernel-replay profiler).

    python -m luatorch_b200.tools.step_profile --preset gpt124m --steps 4

Uses the CUPTI activity records that torch.profiler collects: one line per kernel family with
launches per step, time per step, share of the GPU-busy time and mean duration, plus the span
of a step and the idle gaps between kernels.  The records cost a little host time per launch,
so use the table for SHARES; throughput numbers come from bench.py, which runs unprofiled
(and with programmatic dependent launch on, which this tool switches off for attribution).
(The reference has no counterpart: its tools/benchmark.lua times whole ops with os.clock().)
"""
from __future__ import annotations

import argparse
import collections
import os
import re
import sys

# With programmatic dependent launch a kernel's recorded duration includes the time it spends
# waiting for its predecessor, which makes per-kernel shares meaningless; the breakdown is
# therefore taken in plain stream order unless the caller sets LT_PDL explicitly.
os.environ.setdefault("LT_PDL", "0")

import torch

import luatorch_b200 as lf
from luatorch_b200.train.gpt import PRESETS


def family(name: str) -> str:
    m = re.search(r"(\w+)(<[^(]*)?\(", name)
    base = m.group(1) if m else name[:40]
    t = re.search(r"<([^>]*)>", name)
    return base + ("<" + t.group(1)[:24] + ">" if t else "")


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--preset", default="gpt124m", choices=sorted(PRESETS))
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--top", type=int, default=28)
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print("step_profile needs a GPU")
        return 1
    from torch.profiler import ProfilerActivity, profile

    c = PRESETS[args.preset]
    lf.manual_seed(0)
    model = lf.models.GPT(c["vocab_size"], c["embed_dim"], c["num_heads"], c["num_layers"],
                          c["max_seq_len"], 0.0, pos="learned")
    ddp = lf.distributed.DDP(model)
    opt = lf.optim.AdamW(ddp.parameters(), c["lr"], 0.9, 0.95, 1e-8, c["weight_decay"],
                         model.no_decay_params())
    ddp.attach(opt)
    crit = lf.nn.CrossEntropyLoss(c["vocab_size"], inplace_backward=True)
    tok = torch.randint(0, c["vocab_size"], (c["batch_size"], c["seq_len"] + 1), dtype=torch.int32).cuda()
    x = lf.Tensor.wrap(tok[:, :-1].contiguous())
    y = lf.Tensor.wrap(tok[:, 1:].contiguous().reshape(-1))

    def step():
        lf.autograd.zero_graph()
        ddp.zero_grad()
        loss = crit(ddp(x), y)
        lf.autograd.backward(loss)
        ddp.sync_gradients()
        opt.step()

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(args.steps):
            step()
        torch.cuda.synchronize()
    evs = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA]
    evs.sort(key=lambda e: e.time_range.start)
    agg = collections.defaultdict(lambda: [0, 0.0])
    busy = 0.0
    for e in evs:
        d = e.time_range.end - e.time_range.start
        k = family(e.name)
        agg[k][0] += 1
        agg[k][1] += d
        busy += d
    n = args.steps
    span = evs[-1].time_range.end - evs[0].time_range.start
    print("preset %s: span %.3f ms/step, GPU busy %.3f ms/step, idle gaps %.3f ms/step, %d kernels/step"
          % (args.preset, span / n / 1e3, busy / n / 1e3, (span - busy) / n / 1e3, len(evs) // n))
    for k, (cnt, v) in sorted(agg.items(), key=lambda kv: -kv[1][1])[: args.top]:
        print("%-58s n=%4d %8.3f ms/step %5.1f%% avg %7.1f us"
              % (k[:58], cnt // n, v / n / 1e3, 100 * v / busy, v / cnt))
    return 0


if __name__ == "__main__":
    sys.exit(main())
