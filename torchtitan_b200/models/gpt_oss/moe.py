"""gpt-oss experts: fused gate/up projection with biases and the clamped, interleaved SwiGLU.

Parity: torchtitan/models/gpt_oss/moe.py:23-296. ``mlp1`` produces 2H features with gate and linear
parts interleaved (even / odd); activation = ``min(g, limit) * sigmoid(1.702 * g) * (clamp(l, +-limit) + 1)``.
Under tensor parallel the second bias is divided by the TP degree in forward only
(:class:`ScaleBiasForward`) so that the row-parallel sum adds it exactly once."""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn

from torchtitan_b200.models.common.moe.moe import LocalDispatcher, MoE, _moe_ops
from torchtitan_b200.protocols.module import Module


class ScaleBiasForward(torch.autograd.Function):
    @staticmethod
    def forward(ctx, bias, tp_degree):
        return bias / tp_degree if tp_degree > 1 else bias

    @staticmethod
    def backward(ctx, g):
        return g, None


def swiglu(x, alpha: float = 1.702, limit: float = 7.0):
    g, lin = x[..., ::2], x[..., 1::2]
    g = g.clamp(max=limit)
    lin = lin.clamp(min=-limit, max=limit)
    return g * torch.sigmoid(alpha * g) * (lin + 1)


def _rows_of(per_expert: torch.Tensor, counts: torch.Tensor, rows: int) -> torch.Tensor:
    """Expand per-expert vectors to one per row; rows past ``sum(counts)`` get zeros."""
    slack = (rows - counts.sum()).reshape(1).to(counts.dtype)
    padded = torch.cat((per_expert, per_expert.new_zeros(1, per_expert.shape[-1])))
    return padded.repeat_interleave(torch.cat((counts, slack)).long(), dim=0, output_size=rows)


class GptOssGroupedExperts(Module):
    def __init__(self, *, dim: int, hidden_dim: int, num_experts: int, use_grouped_mm: bool, swiglu_limit: float):
        super().__init__()
        self.num_experts, self.use_grouped_mm, self.swiglu_limit = num_experts, use_grouped_mm, swiglu_limit
        self.mlp1_weight = nn.Parameter(torch.empty(num_experts, hidden_dim * 2, dim))
        self.mlp1_bias = nn.Parameter(torch.empty(num_experts, hidden_dim * 2))
        self.mlp2_weight = nn.Parameter(torch.empty(num_experts, dim, hidden_dim))
        self.mlp2_bias = nn.Parameter(torch.empty(num_experts, dim))
        self.dispatcher = LocalDispatcher()
        self.tp_degree = 1  # set by the tensor-parallel plan
        self.quant = None

    def forward(self, x, num_tokens_per_expert):
        w1, b1, w2, b2 = (p.to_local() if hasattr(p, "to_local") else p
                          for p in (self.mlp1_weight, self.mlp1_bias, self.mlp2_weight, self.mlp2_bias))
        mo = _moe_ops()
        rows = x.shape[0]
        h = mo.grouped_linear(x, w1, num_tokens_per_expert) + _rows_of(b1, num_tokens_per_expert, rows).to(x.dtype)
        h = swiglu(h, limit=self.swiglu_limit)
        b2r = ScaleBiasForward.apply(_rows_of(b2, num_tokens_per_expert, rows), self.tp_degree)
        return mo.grouped_linear(h, w2, num_tokens_per_expert) + b2r.to(h.dtype)

    def init_weights(self, **kwargs) -> None:
        init_std = kwargs.get("init_std")
        assert init_std is not None
        for p in (self.mlp1_weight, self.mlp1_bias, self.mlp2_weight, self.mlp2_bias):
            nn.init.trunc_normal_(p, mean=0.0, std=init_std)


class GptOssMoE(MoE):
    @dataclass(kw_only=True, slots=True)
    class Config(MoE.Config):
        swiglu_limit: float = 7.0

    def __init__(self, config: Config, *, dim: int):
        super().__init__(config, dim=dim)
        self.experts = GptOssGroupedExperts(dim=dim, hidden_dim=config.hidden_dim, num_experts=config.num_experts,
                                            use_grouped_mm=config.use_grouped_mm, swiglu_limit=config.swiglu_limit)
