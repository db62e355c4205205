"""Loss builders. The training loss is the *sum* of token cross-entropies (fp32, labels equal
to ``IGNORE_INDEX`` contribute nothing); the Trainer divides by the global number of valid
tokens. Parity: torchtitan/components/loss.py:16-53."""

from __future__ import annotations

from typing import Callable

import torch

from torchtitan_b200 import ops

IGNORE_INDEX = -100

LossFunction = Callable[..., torch.Tensor]


def cross_entropy_loss(pred: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
    group = getattr(pred, "_tp_vocab_sharded", None)
    if group is not None:  # logits are sharded over the vocabulary (tensor parallel + loss parallel)
        from torchtitan_b200.parallel.tp import vocab_parallel_cross_entropy_sum

        return vocab_parallel_cross_entropy_sum(pred, labels, group, IGNORE_INDEX)
    return ops.cross_entropy_sum(pred, labels, IGNORE_INDEX)


def build_cross_entropy_loss(compile_config=None, **kwargs) -> LossFunction:
    # compile_config is accepted for API parity; the CUDA path is already one fused kernel
    return cross_entropy_loss


def mse_loss(pred: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
    return torch.nn.functional.mse_loss(pred.float(), labels.float().detach(), reduction="sum")


def build_mse_loss(compile_config=None, **kwargs) -> LossFunction:
    return mse_loss
