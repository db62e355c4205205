"""Model converters rewrite a freshly built (meta-device) model, e.g. swap ``Linear`` for a
quantised variant, and may run a hook after every optimizer step.

Parity: torchtitan/protocols/model_converter.py:17-101 (container builds each converter
config with ``parallel_dims`` and ``model_compile_enabled``; two converters of different
quantisation families in one job are rejected).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Protocol

import torch.nn as nn

from torchtitan_b200.config.configurable import Configurable


class ModelConverter(Protocol):
    def convert(self, model: nn.Module): ...

    def post_optimizer_hook(self, model: nn.Module | list[nn.Module]): ...


def _validate_quantization(converters: list) -> None:
    kinds = {}
    for c in converters:
        owner = type(c)._owner
        kind = getattr(type(c), "_quantization_type", None) or getattr(owner, "_quantization_type", None)
        if kind is not None:
            kinds.setdefault(kind, []).append(owner.__name__)
    if len(kinds) > 1:
        raise ValueError(
            "Cannot combine model converters with different quantization types: "
            + ", ".join(f"{k}={v}" for k, v in kinds.items())
        )


class ModelConvertersContainer(Configurable, ModelConverter):
    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        converters: list = field(default_factory=list)
        """Converter ``Config`` objects, applied in order."""
        print_after_conversion: bool = False

    def __init__(self, config: Config, *, parallel_dims, model_compile_enabled: bool = False):
        _validate_quantization(config.converters)
        self.converters = [
            c.build(parallel_dims=parallel_dims, model_compile_enabled=model_compile_enabled)
            for c in config.converters
        ]
        self.print_after_conversion = config.print_after_conversion

    def convert(self, model: nn.Module):
        for c in self.converters:
            c.convert(model)
        if self.print_after_conversion:
            from torchtitan_b200.tools.logging import logger

            logger.info(f"Model definition after conversion:\n\n{model}\n\n")

    def post_optimizer_hook(self, model: nn.Module | list[nn.Module]):
        for c in self.converters:
            c.post_optimizer_hook(model)
