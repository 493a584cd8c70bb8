"""Training entry points (counterparts of the reference's examples/xor.lua, mnist.lua,
cifar.lua and gpt.lua):

    python -m luatorch_b200.train.xor                      # CPU, fp32
    python -m luatorch_b200.train.mlp  [--steps N]         # MLP classifier, data parallel
    python -m luatorch_b200.train.convnet [--steps N]      # conv net, data parallel
    python -m luatorch_b200.train.gpt  [--preset gpt124m]  # GPT, fused all-reduce + AdamW

Multi-GPU: launch with `python -m torch.distributed.run --nproc-per-node N -m luatorch_b200.train.gpt`.
"""
