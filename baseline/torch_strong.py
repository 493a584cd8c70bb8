"""Strong baseline: the same GPT training step written with stock PyTorch modules, so the
framework's numbers can be read against the library stack on the same box (cuBLAS GEMMs,
the fused scaled_dot_product_attention kernels, torch.optim.AdamW(fused=True), bucketed
DistributedDataParallel over NCCL).  None of this repository's kernels run here.

    python baseline/torch_strong.py --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29533 baseline/torch_strong.py --gpus 8 --steps 20 --warmup 5

Model: the reference's GPT (lua/luatorch/models/gpt.lua:36-54, 62-93) at the GPT-124M
configuration: token embedding + learned positions, 12 pre-LayerNorm blocks (q/k/v without
bias, out-projection with bias, GELU(tanh) feed-forward x4), final LayerNorm, untied head
without bias; bf16 autocast with fp32 master weights, AdamW lr 6e-4 wd 0.1 (no decay on
LayerNorm parameters and biases), synthetic uniform tokens, CUDA-event timing, max over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.nn as nn
import torch.nn.functional as F


class Block(nn.Module):
    def __init__(self, e, h):
        super().__init__()
        self.h = h
        self.ln1, self.ln2 = nn.LayerNorm(e), nn.LayerNorm(e)
        self.qkv = nn.Linear(e, 3 * e, bias=False)
        self.out = nn.Linear(e, e)
        self.ffn1, self.ffn2 = nn.Linear(e, 4 * e), nn.Linear(4 * e, e)

    def forward(self, x):
        b, s, e = x.shape
        q, k, v = self.qkv(self.ln1(x)).view(b, s, 3, self.h, e // self.h).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        x = x + self.out(a.transpose(1, 2).reshape(b, s, e))
        return x + self.ffn2(F.gelu(self.ffn1(self.ln2(x)), approximate="tanh"))


class GPT(nn.Module):
    def __init__(self, vocab, e, h, layers, max_seq):
        super().__init__()
        self.tok, self.pos = nn.Embedding(vocab, e), nn.Embedding(max_seq, e)
        self.blocks = nn.ModuleList(Block(e, h) for _ in range(layers))
        self.ln = nn.LayerNorm(e)
        self.head = nn.Linear(e, vocab, bias=False)

    def forward(self, idx):
        s = idx.shape[1]
        x = self.tok(idx) + self.pos(torch.arange(s, device=idx.device))
        for blk in self.blocks:
            x = blk(x)
        return self.head(self.ln(x))


PRESETS = {"124M": dict(vocab=50257, e=768, h=12, layers=12, seq=1024, mb=8),
           "1.3B": dict(vocab=50257, e=2048, h=16, layers=24, seq=2048, mb=4)}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--model", default="124M", choices=sorted(PRESETS))
    args = ap.parse_args(argv)
    cfg = PRESETS[args.model]
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        torch.distributed.init_process_group("nccl", device_id=dev)
    torch.manual_seed(1234)
    model = GPT(cfg["vocab"], cfg["e"], cfg["h"], cfg["layers"], cfg["seq"]).to(dev)
    decay = [p for n, p in model.named_parameters() if p.dim() >= 2]
    no_decay = [p for n, p in model.named_parameters() if p.dim() < 2]
    opt = torch.optim.AdamW([{"params": decay, "weight_decay": 0.1},
                             {"params": no_decay, "weight_decay": 0.0}], lr=6e-4, fused=True)
    net = model
    if world > 1:
        net = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local],
                                                        gradient_as_bucket_view=True)
    g = torch.Generator(device=dev).manual_seed(99 + rank)
    tokens = torch.randint(0, cfg["vocab"], (cfg["mb"], cfg["seq"] + 1), device=dev, generator=g)
    x, y = tokens[:, :-1].contiguous(), tokens[:, 1:].contiguous()

    def step():
        with torch.autocast("cuda", dtype=torch.bfloat16):
            logits = net(x)
        loss = F.cross_entropy(logits.float().view(-1, cfg["vocab"]), y.view(-1))
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss

    for _ in range(max(3, args.warmup)):
        step()
    if world > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        loss = step()
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        torch.distributed.all_reduce(ms, op=torch.distributed.ReduceOp.MAX)
    if rank == 0:
        per = ms.item() / args.steps
        print(json.dumps({"impl": "torch_strong", "model": args.model, "n_gpus": world,
                          "ms_per_step": per, "value": cfg["mb"] * cfg["seq"] * world / (per * 1e-3),
                          "unit": "tokens/s", "steps": args.steps, "dtype": "bf16 autocast, fp32 master",
                          "final_loss": float(loss), "mem_gb": torch.cuda.max_memory_allocated() / 2**30}),
              flush=True)
    if world > 1:
        torch.distributed.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
