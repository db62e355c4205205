"""SwiGLU feed-forward: ``w2(silu(w1 x) * w3 x)``.

Parity: torchtitan/models/common/feed_forward.py:18-67 (``hidden_dim`` in the config is final;
``compute_ffn_hidden_dim`` applies the Llama 2/3 * 4 * dim rule with multiplier and rounding).
"""

from dataclasses import dataclass, field

from torchtitan_b200 import ops
from torchtitan_b200.protocols.module import Module

from .linear import Linear, project_together


def compute_ffn_hidden_dim(dim: int, *, multiple_of: int = 1, ffn_dim_multiplier: float | None = None) -> int:
    hidden = int(2 * 4 * dim / 3)
    if ffn_dim_multiplier is not None:
        hidden = int(ffn_dim_multiplier * hidden)
    return multiple_of * -(-hidden // multiple_of)


class FeedForward(Module):
    @dataclass(kw_only=True, slots=True)
    class Config(Module.Config):
        hidden_dim: int
        linear_bias: bool = False
        dim: int = field(init=False)

    def __init__(self, config: Config):
        super().__init__()
        lin = Linear.Config(bias=config.linear_bias)
        self.w1 = lin.build(in_features=config.dim, out_features=config.hidden_dim)
        self.w2 = lin.build(in_features=config.hidden_dim, out_features=config.dim)
        self.w3 = lin.build(in_features=config.dim, out_features=config.hidden_dim)

    def forward(self, x, residual=None):
        """``w2(silu(w1 x) * w3 x)``, plus ``residual`` (the block's skip connection) when given."""
        h = ops.swiglu(*project_together(x, self.w1, self.w3))
        return self.w2(h) if residual is None else self.w2.add_to(residual, h)

    def init_weights(self, init_std: float = 0.02, **kwargs):
        self.w1.init_weights()
        self.w2.init_weights(init_std=init_std)
        self.w3.init_weights(init_std=init_std)
