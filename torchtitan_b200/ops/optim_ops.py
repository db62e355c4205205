"""Flat-buffer optimizer math: AdamW over one contiguous shard and squared-norm partials."""

from __future__ import annotations

import math

import torch


def adamw_flat(param, grad, exp_avg, exp_avg_sq, shadow, *, lr, beta1, beta2, eps, weight_decay, step,
               decoupled=True, grad_scale=None):
    """In-place AdamW on flat fp32 buffers; ``shadow`` (optional, compute dtype) receives the
    updated parameters; ``grad_scale`` (python float or 0-dim tensor) multiplies the gradient
    first (used to fold gradient clipping into the same pass)."""
    if param.is_cuda:
        from . import cuda_ops

        return cuda_ops.adamw_flat(param, grad, exp_avg, exp_avg_sq, shadow, lr=lr, beta1=beta1, beta2=beta2,
                                   eps=eps, weight_decay=weight_decay, step=step, decoupled=decoupled,
                                   grad_scale=grad_scale)
    g = grad if grad_scale is None else grad * grad_scale
    if decoupled:
        param.mul_(1 - lr * weight_decay)
    elif weight_decay != 0:
        g = g.add(param, alpha=weight_decay)
    exp_avg.lerp_(g, 1 - beta1)
    exp_avg_sq.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    bc1 = 1 - beta1**step
    bc2 = 1 - beta2**step
    denom = (exp_avg_sq.sqrt() / math.sqrt(bc2)).add_(eps)
    param.addcdiv_(exp_avg, denom, value=-lr / bc1)
    if shadow is not None:
        shadow.copy_(param)


def sumsq(flat) -> torch.Tensor:
    """fp32 sum of squares of a flat buffer (0-dim tensor on the same device)."""
    if flat.is_cuda:
        from . import cuda_ops

        return cuda_ops.sumsq(flat)
    return flat.float().pow(2).sum()
