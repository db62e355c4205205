"""``RMSNorm`` (state-dict compatible with ``nn.RMSNorm``); forward is the fused fp32-math
kernel on GPU. Parity: torchtitan/models/common/rmsnorm.py:14-50."""

from dataclasses import dataclass, field

import torch.nn as nn

from torchtitan_b200 import ops
from torchtitan_b200.protocols.module import Module


class RMSNorm(nn.RMSNorm, Module):
    @dataclass(kw_only=True, slots=True)
    class Config(Module.Config):
        normalized_shape: int = field(init=False)
        eps: float = 1e-5
        elementwise_affine: bool = True

    def __init__(self, config: Config):
        if not hasattr(config, "normalized_shape"):
            raise TypeError(
                "RMSNorm.Config requires 'normalized_shape' to be set (use Config.build(normalized_shape=...))."
            )
        super().__init__(config.normalized_shape, eps=config.eps, elementwise_affine=config.elementwise_affine)
        self.config = config

    def forward(self, x):
        return ops.rms_norm(x, self.weight, self.eps)

    def init_weights(self, **kwargs) -> None:
        self.reset_parameters()
