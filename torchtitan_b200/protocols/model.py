"""``BaseModel``: root of trainable models; its ``Config`` can read the job config and count
parameters and FLOPs. Parity: torchtitan/protocols/model.py:13-43."""

from abc import abstractmethod
from dataclasses import dataclass

import torch.nn as nn

from .module import Module


class BaseModel(Module):
    @dataclass(kw_only=True, slots=True)
    class Config(Module.Config):
        @abstractmethod
        def update_from_config(self, *, trainer_config, **kwargs) -> None:
            """Adapt the model config to the job (sequence length, parallel degrees, ...)."""

        @abstractmethod
        def get_nparams_and_flops(self, model: nn.Module, seq_len: int) -> tuple[int, int]:
            """Return (parameter count, training FLOPs per token)."""
