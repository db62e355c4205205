"""``Linear``: an ``nn.Linear`` (same parameter names and state dict) whose forward runs the
framework GEMM. Parity: torchtitan/models/common/linear.py:14-56 (late-bound in/out
features, truncated-normal init with a per-call ``init_std`` override, zero bias)."""

from dataclasses import dataclass, field

import torch.nn as nn

from torchtitan_b200 import ops
from torchtitan_b200.protocols.module import Module


class Linear(nn.Linear, Module):
    @dataclass(kw_only=True, slots=True)
    class Config(Module.Config):
        in_features: int = field(init=False)
        out_features: int = field(init=False)
        bias: bool = False
        init_mean: float = 0.0
        init_std: float = 0.02

    def __init__(self, config: Config):
        if not (hasattr(config, "in_features") and hasattr(config, "out_features")):
            raise TypeError(
                "Linear.Config requires 'in_features' and 'out_features' to be set "
                "(use Config.build(in_features=..., out_features=...))."
            )
        super().__init__(config.in_features, config.out_features, bias=config.bias)
        self._init_mean, self._init_std = config.init_mean, config.init_std
        self.quant = None  # a QuantRecipe once a quantisation converter selected this layer

    def forward(self, x):
        if self.quant is not None:
            from torchtitan_b200.ops.quant import quant_linear

            return quant_linear(x, self.weight, self.bias, self.quant)
        return ops.linear(x, self.weight, self.bias)

    def init_weights(self, **kwargs) -> None:
        std = kwargs.get("init_std")
        nn.init.trunc_normal_(self.weight, mean=self._init_mean, std=self._init_std if std is None else std)
        if self.bias is not None:
            nn.init.zeros_(self.bias)
