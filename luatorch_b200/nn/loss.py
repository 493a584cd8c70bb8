"""Loss layers MSELoss / MAELoss / CrossEntropyLoss (lua/luatorch/nn/loss.lua).

Each returns a [1] fp32 tensor on the prediction's device.  Unlike the reference, whose
backward closures ignore the incoming gradient (loss.lua:16-26, 71-81), the upstream gradient
multiplies the result, so scaled losses (GradScaler) propagate correctly.  On CUDA the cross
entropy is the fused softmax-CE pair: forward saves the row log-sum-exp, backward reads the
logits once and may overwrite them with the gradient."""
from __future__ import annotations


from .. import _backend as B
from ..utils import debug as _debug
from .. import autograd
from ..tensor import Tensor
from .module import Module


def _upstream_scale(g: Tensor):
    """(host scale, device scale tensor or None) for an incoming loss gradient."""
    if getattr(g, "_unit", False):
        return 1.0, None
    if g._t.is_cuda:
        return 1.0, g._t.reshape(-1)[:1].float()
    return float(g._t.reshape(-1)[0]), None


class _PointwiseLoss(Module):
    mode = 0

    def forward(self, pred: Tensor, target: Tensor) -> Tensor:
        fwd = B.mse_loss if self.mode == 0 else B.mae_loss
        bwd = B.mse_loss_backward if self.mode == 0 else B.mae_loss_backward
        out = Tensor(_data=fwd(pred._t, target._t))

        def grad_fn(g):
            if pred.requires_grad:
                s, dev = _upstream_scale(g)
                grad = bwd(pred._t, target._t, s)
                if dev is not None:
                    grad = B.binary("mul", grad, dev.to(grad.dtype).expand(grad.numel()).contiguous())
                autograd.acc_grad(pred, grad)

        autograd.record("mse_loss" if self.mode == 0 else "mae_loss", [pred], out, grad_fn)
        return out


class MSELoss(_PointwiseLoss):
    mode = 0


class MAELoss(_PointwiseLoss):
    mode = 1


class CrossEntropyLoss(Module):
    """Mean cross entropy of raw logits [batch, classes] against class labels [batch]."""

    def __init__(self, n_classes: int = None, inplace_backward: bool = False):
        self.n_classes = n_classes          # logical class count when logits are column padded
        self.inplace_backward = inplace_backward

    def forward(self, pred: Tensor, target: Tensor) -> Tensor:
        logits = pred._t
        labels = target._t
        cols = self.n_classes or logits.shape[1]
        if logits.is_cuda:
            if not labels.is_cuda:
                labels = labels.cuda()
            fused = (self.inplace_backward and autograd.enabled and pred.requires_grad
                     and logits.stride(-1) == 1)
            if fused:
                # one kernel: loss, log-sum-exp, and the logits overwritten by their gradient
                # for an upstream gradient of 1 (rescaled in backward if it is not)
                loss, lse, err = B.ext().cross_entropy_fused(logits, cols, B._labels(labels),
                                                              1.0 / logits.shape[0])
            else:
                loss, lse, err = B.cross_entropy_device(logits, labels, cols)
            self.last_error_flag = err
            _debug.check_index_word(err, "CrossEntropyLoss: label")
        else:
            r = B.cross_entropy_full(logits, labels, cols)
            if r is None:
                import sys
                print("luatorch error: cross_entropy_loss label out of range", file=sys.stderr)
                return None
            loss, lse = r
        out = Tensor(_data=loss)
        inplace = self.inplace_backward

        fused_done = logits.is_cuda and fused

        def grad_fn(g):
            if pred.requires_grad:
                s, dev = _upstream_scale(g)
                if fused_done:
                    dl = logits                      # already (softmax - onehot) / rows
                    if dev is not None:
                        dl[:, :cols].mul_(dev * s)
                    elif s != 1.0:
                        dl[:, :cols].mul_(s)
                else:
                    dl = B.cross_entropy_backward(logits, labels, lse, s,
                                                  out=logits if inplace else None,
                                                  n_classes=cols, scale_dev=dev)
                autograd.acc_grad(pred, dl)

        autograd.record("cross_entropy_loss", [pred], out, grad_fn)
        return out
