"""`lf.ops`: the functional kernel layer, for code that builds its own layers.

Every function takes and returns `torch.Tensor`s (use `Tensor._t` / `Tensor.wrap` to cross to
the tape-recording `lf.Tensor` world) and dispatches on the device: on CUDA to this package's
sm_100a kernels (csrc/kernels/), on CPU to plain fp32 tensor math with the same semantics.  None
of them records autograd; the `nn` modules pair each forward with its backward.

    gemm                      C = act(alpha * op(A) @ op(B) + bias) + residual   (tcgen05; every
                              transposed form, bias / GELU / dGELU / ReLU / residual / accumulate
                              epilogues, split-K) - replaces cublasSgemm (csrc/cuda/ops/matmul.cu:92-141)
    matmul, bmm, transpose, dot
    layernorm / layernorm_backward          csrc/cuda/ops/fused.cu:63-127 (the reference has no backward)
    gelu_bias / gelu_bias_backward          csrc/cuda/ops/fused.cu:26-58
    softmax, cross_entropy / cross_entropy_backward     csrc/cuda/ops/loss.cu:14-125
    attention_forward / attention_backward  causal flash attention, [B, S, H, D] views
                                            (csrc/cuda/ops/flash_attention.cu:19-145 is forward only)
    dropout / dropout_backward              mask regenerated from a Philox (seed, offset) pair
    im2col / col2im, relayout               convolution lowering
    add_broadcast / column_sum              bias add and its gradient
    adamw_flat / sgd_flat                   one launch over a flat parameter arena
    gather_matmul                           all-gather of a row-sharded weight fused into the GEMM
"""
from .._backend import (add_broadcast, adamw_flat, attention_backward, attention_forward, bmm, cast,
                        col2im, column_sum, cross_entropy, cross_entropy_backward, dot, dropout,
                        dropout_backward, gelu_bias, gelu_bias_backward, gemm, im2col, layernorm,
                        layernorm_backward, matmul, relayout, sgd_flat, softmax, transpose)


def gather_matmul(*args, **kwargs):
    """See `luatorch_b200.distributed.gather_matmul` (imported lazily: it needs the process group)."""
    from ..distributed import gather_matmul as _gm
    return _gm(*args, **kwargs)


__all__ = ["add_broadcast", "adamw_flat", "attention_backward", "attention_forward", "bmm", "cast",
           "col2im", "column_sum", "cross_entropy", "cross_entropy_backward", "dot", "dropout",
           "dropout_backward", "gelu_bias", "gelu_bias_backward", "gemm", "im2col", "layernorm",
           "layernorm_backward", "matmul", "relayout", "sgd_flat", "softmax", "transpose",
           "gather_matmul"]
