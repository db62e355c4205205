"""Warmup -> (stable) -> decay learning-rate schedule applied to every optimizer.

Parity: torchtitan/components/lr_scheduler.py:50-228. The multiplier at step ``s``
(``LambdaLR`` semantics, ``s`` = number of ``step()`` calls so far):

* warmup: ``(s + 1) / warmup_steps`` (the last warm-up step already runs at the full rate);
* stable: 1 for ``stable_steps = total + 1 - warmup - decay`` steps (the ``+ 1`` is a virtual
  last step so the rate never reaches ``min_lr_factor`` exactly inside training);
* decay over ``decay_steps = decay_ratio * total`` (or everything after warmup when
  ``decay_ratio is None``): progress ``(s + 1 - warmup - stable) / decay``, remaining fraction
  ``1 - progress`` (``linear``), ``1 - sqrt(progress)`` (``sqrt``) or the cosine half period
  (``cosine``), then mapped to ``[min_lr_factor, 1]``.

``total`` defaults to ``training.steps``; too-long warmup/decay are clipped with a warning.
Only the first scheduler's state is checkpointed (all are identical).
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Callable, Iterator, Literal

from torch.distributed.checkpoint.stateful import Stateful
from torch.optim.lr_scheduler import LambdaLR, LRScheduler

from torchtitan_b200.config.configurable import Configurable
from torchtitan_b200.tools.logging import logger

__all__ = ["LRSchedulersContainer", "wsd_multiplier"]


def wsd_multiplier(step: int, *, warmup: int, stable: int, decay: int, kind: str, floor: float) -> float:
    if step < warmup:
        return float((step + 1) / warmup)
    if step < warmup + stable:
        return 1.0
    assert decay != 0, "decay_steps must not be zero to reach the decay phase"
    progress = float(step + 1 - warmup - stable) / decay
    if kind == "linear":
        f = 1.0 - progress
    elif kind == "sqrt":
        f = 1.0 - math.sqrt(progress)
    elif kind == "cosine":
        f = 0.5 * (1.0 + math.cos(math.pi * progress))
    else:
        raise ValueError(f"unknown lr decay type {kind}")
    return floor + (1.0 - floor) * f


class LRSchedulersContainer(Stateful, Configurable):
    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        warmup_steps: int = 200
        decay_ratio: float | None = None
        """Fraction of total steps spent decaying; None = decay right after warmup (no plateau)."""
        decay_type: Literal["linear", "sqrt", "cosine"] = "linear"
        min_lr_factor: float = 0.0
        total_steps: int | None = None
        """Length of the schedule if different from training.steps."""

    schedulers: list[LRScheduler]

    def __init__(self, config: Config | None = None, *, optimizers=None, training_steps: int | None = None,
                 lr_lambda: Callable | None = None):
        assert optimizers is not None and len(optimizers) > 0, "Must have at least one optimizer to create LRScheduler"
        if lr_lambda is None:
            lr_lambda = self._make_lambda(config, training_steps)
        self.schedulers = [LambdaLR(opt, lr_lambda) for opt in optimizers]

    @staticmethod
    def _make_lambda(config: "LRSchedulersContainer.Config", training_steps: int) -> Callable[[int], float]:
        total = config.total_steps if config.total_steps is not None else training_steps
        warmup = int(config.warmup_steps)
        if warmup > total:
            logger.warning(f"Warmup steps ({warmup}) exceed total training steps ({total}). Adjusting warmup steps to {total}.")
            warmup = total
        if config.decay_ratio is not None:
            decay = round(total * config.decay_ratio)
            if warmup + decay > total:
                logger.warning(
                    f"Warmup ({warmup}) + decay ({decay}) steps exceed total training steps ({total}). "
                    f"Adjusting decay steps to {total - warmup}."
                )
                decay = total - warmup
        else:
            decay = total - warmup
        stable = total + 1 - warmup - decay
        kind, floor = config.decay_type, config.min_lr_factor

        def fn(step: int) -> float:
            return wsd_multiplier(step, warmup=warmup, stable=stable, decay=decay, kind=kind, floor=floor)

        return fn

    def __iter__(self) -> Iterator[LRScheduler]:
        return iter(self.schedulers)

    def __len__(self) -> int:
        return len(self.schedulers)

    def step(self) -> None:
        for s in self.schedulers:
            s.step()

    def state_dict(self) -> dict[str, Any]:
        return self.schedulers[0].state_dict()

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        import copy

        for s in self.schedulers:
            s.load_state_dict(copy.deepcopy(state_dict))
