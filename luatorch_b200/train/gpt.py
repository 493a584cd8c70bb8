"""GPT training, data parallel with the fused all-reduce + AdamW (counterpart of the
reference's examples/gpt.lua, same configuration keys: embed_dim, num_heads, num_layers,
max_seq_len, dropout, batch_size, seq_len, lr, weight_decay, warmup_steps, max_steps, use_amp,
use_ddp, export_onnx, print_every, sample_every, save_every, temperature, top_k, gen_tokens).

    python -m luatorch_b200.train.gpt --preset small --text corpus.txt
    python -m torch.distributed.run --nproc-per-node 8 -m luatorch_b200.train.gpt --preset gpt124m
    ... --preset gpt1p3b --mode sharded      # sharded optimizer state (reduce-scatter + shard AdamW)

Without --text the tokens are synthetic (uniform over the vocabulary).  Throughput is timed on
the device with CUDA events.

`use_amp` (examples/gpt.lua:113-118,170-174 in the reference) trains through a `GradScaler`:
the loss is scaled before backward, the averaged gradients are checked for inf / nan on the
device, and the optimizer launch skips itself on overflow.  The gradient reduction then runs
unfused (the skip decision needs the reduced gradients), with full-length optimizer state.
"""
from __future__ import annotations

import argparse

import torch

import luatorch_b200 as lf
from .common import StepTimer, log

PRESETS = {
    "small": dict(vocab_size=256, embed_dim=384, num_heads=6, num_layers=6, max_seq_len=128, seq_len=128,
                  batch_size=4, lr=3e-4, weight_decay=0.01),
    "gpt124m": dict(vocab_size=50257, embed_dim=768, num_heads=12, num_layers=12, max_seq_len=1024, seq_len=1024,
                    batch_size=8, lr=6e-4, weight_decay=0.1),
    "gpt1p3b": dict(vocab_size=50257, embed_dim=2048, num_heads=16, num_layers=24, max_seq_len=2048, seq_len=2048,
                    batch_size=4, lr=2e-4, weight_decay=0.1),
}
DEFAULTS = dict(dropout=0.0, warmup_steps=100, max_steps=200, use_amp=False, use_ddp=True, export_onnx=False,
                print_every=10, sample_every=0, save_every=0, temperature=0.8, top_k=40, gen_tokens=100)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--preset", default="small", choices=sorted(PRESETS))
    ap.add_argument("--config", default="", help="JSON or `return { ... }` Lua-table file overriding the preset")
    ap.add_argument("--text", default="", help="training text file (character level); synthetic tokens if empty")
    ap.add_argument("--mode", default="sharded", choices=["sharded", "replicated", "nccl"])
    ap.add_argument("--max-steps", type=int, default=0)
    ap.add_argument("--out", default="", help="checkpoint path (.bin)")
    ap.add_argument("--bucket-mb", type=float, default=32.0)
    ap.add_argument("--graph", action="store_true",
                    help="replay the step as a CUDA graph (two extra warm-up steps)")
    ap.add_argument("--amp", action="store_true", help="same as use_amp = true in the config")
    ap.add_argument("--resume", default="", help="checkpoint path (.bin) to resume from")
    args = ap.parse_args(argv)
    cfg = lf.utils.Config({**DEFAULTS, **PRESETS[args.preset]})
    if args.config:
        cfg.load(args.config)
    if args.max_steps:
        cfg.set("max_steps", args.max_steps)
    if args.amp:
        cfg.set("use_amp", True)
    lf.distributed.init()
    rank, world = lf.distributed.rank(), lf.distributed.world_size()
    if rank == 0:
        cfg.print()
    lf.manual_seed(1234)
    cuda = torch.cuda.is_available()
    dev = "cuda" if cuda else "cpu"
    dataset = None
    if args.text:
        dataset = lf.data.TextDataset(args.text, cfg.get("seq_len"), "train", verbose=rank == 0)
        cfg.set("vocab_size", dataset.vocab_size)
    V, S, Bm = cfg.get("vocab_size"), cfg.get("seq_len"), cfg.get("batch_size")
    model = lf.models.GPT(V, cfg.get("embed_dim"), cfg.get("num_heads"), cfg.get("num_layers"),
                          cfg.get("max_seq_len"), cfg.get("dropout"), pos="learned")
    log(model)
    use_amp = bool(cfg.get("use_amp")) and cuda
    ddp = lf.distributed.DDP(model, mode=args.mode, bucket_mb=args.bucket_mb, device=dev,
                             shard_state=not use_amp)
    opt = lf.optim.AdamW(ddp.parameters(), cfg.get("lr"), 0.9, 0.95, 1e-8, cfg.get("weight_decay"),
                         model.no_decay_params())
    scaler = lf.cuda.amp.GradScaler() if use_amp else None
    if scaler is None:
        ddp.attach(opt)      # gradient reduction fused with the optimizer update
    sched = lf.optim.WarmupScheduler(opt, cfg.get("warmup_steps"),
                                     lf.optim.CosineAnnealing(opt, max(1, cfg.get("max_steps") - cfg.get("warmup_steps")),
                                                              cfg.get("lr") * 0.1))
    crit = lf.nn.CrossEntropyLoss(V, inplace_backward=cuda)
    logger = lf.utils.Logger(cfg.get("print_every"))
    gen = torch.Generator().manual_seed(4321 + rank)

    def batch():
        if dataset is not None:
            x, y = dataset.get_batch(Bm)
            xt, yt = x._t, y._t.reshape(-1)
        else:
            t = torch.randint(0, V, (Bm, S + 1), generator=gen)
            xt, yt = t[:, :-1].float(), t[:, 1:].reshape(-1).float()
        if cuda:
            xt, yt = xt.pin_memory().to(dev, non_blocking=True), yt.pin_memory().to(dev, non_blocking=True)
        return lf.Tensor.wrap(xt.contiguous()), lf.Tensor.wrap(yt.contiguous())

    x0, y0 = batch()

    def one_step(x=x0, y=y0):
        lf.autograd.zero_graph()
        ddp.zero_grad()
        loss = crit(ddp(x), y)
        if scaler is not None:
            lf.autograd.backward(scaler.scale_loss(loss))
            ddp.sync_gradients()          # averaged over the ranks: every rank takes the same decision
            scaler.step(opt)
            scaler.update()
        else:
            lf.autograd.backward(loss)
            ddp.sync_gradients()
            opt.step()
        return loss

    first_step = 1
    if args.resume:
        meta = ddp.load_checkpoint(args.resume, opt, sched, scaler)
        first_step = int(meta.get("step", 0)) + 1
        log("resumed from %s at step %d" % (args.resume, first_step - 1))
    runner = None
    if args.graph and cuda and scaler is None:
        runner = lf.cuda.GraphedStep(one_step, opt, inputs=(x0, y0), warmup=2)
    timer = StepTimer()
    window = 0
    for step in range(first_step, cfg.get("max_steps") + 1):
        x, y = batch()
        if runner is None and cuda and (step % cfg.get("print_every")) == 0:
            ddp.profile_next_step(True)      # time this step's bucket kernels for the log line
        loss = runner(x, y) if runner is not None else one_step(x, y)
        lr = sched.step()
        window += 1
        if step % cfg.get("print_every") == 0:
            ms = timer.elapsed_ms()
            if rank == 0:
                logger.step = step - 1
                if runner is None and cuda:
                    logger.log_comm(ddp.comm_profile(),
                                    {"allocated_mb": round(lf.Tensor.cuda_memory_allocated() / 1e6, 1),
                                     "cached_mb": round(lf.Tensor.cuda_memory_cached() / 1e6, 1)})
                logger.log(loss.item(), None, lr, tokens=Bm * S * world * window, step_ms=ms)
            ddp.profile_next_step(False)
            ddp.check()
            timer.reset()
            window = 0
        if rank == 0 and cfg.get("sample_every") and step % cfg.get("sample_every") == 0 and dataset is not None:
            prompt = dataset.tokenizer.encode_tensor("The ")
            out = model.generate(prompt, cfg.get("gen_tokens"), cfg.get("temperature"), cfg.get("top_k"))
            print("sample:", repr(dataset.tokenizer.decode_tensor(out)))
        if args.out and cfg.get("save_every") and step % cfg.get("save_every") == 0:
            ddp.save_checkpoint(args.out, opt, sched, scaler, step=step)     # collective
    if args.out:
        ddp.save_checkpoint(args.out, opt, sched, scaler, step=cfg.get("max_steps"))
        log("saved", args.out)
    if rank == 0 and cfg.get("export_onnx") and args.out:
        lf.export.onnx.export(model, lf.Tensor.wrap(torch.zeros(1, min(S, 16)).to(dev)), args.out + ".onnx")
    if cuda:
        log("memory reserved: %.1f MB" % (lf.Tensor.cuda_memory_allocated() / 1e6))
    lf.distributed.destroy()


if __name__ == "__main__":
    main()
