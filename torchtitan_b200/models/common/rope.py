"""Rotary position embedding.

One fp32 table ``[max_seq_len, dim/2, 2]`` holding (cos, sin) per position and frequency
serves both pairing conventions; the ``backend`` only selects which elements of a head form
a rotated pair (``complex`` = adjacent elements, ``cos_sin`` = element i with i + dim/2).
Frequency scaling rules and defaults follow torchtitan/models/common/rope.py:23-209:
``llama`` (factor 8, low/high frequency factors 1/4, original context 8192) and ``yarn``
(NTK-by-parts ramp between ``beta_fast`` and ``beta_slow`` rotations; the cos_sin flavour also
scales cos/sin by ``0.1 ln(factor) + 1``). Tables are indexed by explicit ``positions`` when
given (:212-282), which is how context parallel keeps global positions on a sequence shard.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Literal

import torch

from torchtitan_b200 import ops
from torchtitan_b200.protocols.module import Module


def _yarn_ramp(lo: float, hi: float, n: int) -> torch.Tensor:
    if lo == hi:
        hi += 0.001
    return ((torch.arange(n, dtype=torch.float32) - lo) / (hi - lo)).clamp(0, 1)


class RoPE(Module):
    @dataclass(kw_only=True, slots=True)
    class Config(Module.Config):
        dim: int
        max_seq_len: int
        theta: float = 10000.0
        backend: Literal["complex", "cos_sin"] = "complex"
        scaling: Literal["none", "llama", "yarn"] = "none"
        scaling_factor: float = 8.0
        low_freq_factor: float = 1.0
        high_freq_factor: float = 4.0
        original_max_position_embeddings: int = 8192
        rope_factor: float = 1.0
        beta_fast: float = 32.0
        beta_slow: float = 1.0
        original_seq_len: int = 4096
        mscale: float = 0.0

    def __init__(self, config: Config):
        super().__init__()
        self.config = config
        self.cache = self._precompute()

    @property
    def layout(self) -> str:
        return "interleaved" if self.config.backend == "complex" else "half"

    # ---- frequencies ------------------------------------------------------------
    def inv_freq(self) -> tuple[torch.Tensor, float]:
        """(inverse frequencies [dim/2], magnitude scale applied to cos and sin)."""
        c = self.config
        half = c.dim // 2
        expo = torch.arange(0, c.dim, 2)[:half].float() / c.dim
        if c.backend == "complex":
            f = 1.0 / (c.theta**expo)
            if c.scaling == "llama":
                wavelen = 2 * math.pi / f
                lo_wl = c.original_max_position_embeddings / c.low_freq_factor
                hi_wl = c.original_max_position_embeddings / c.high_freq_factor
                smooth = (c.original_max_position_embeddings / wavelen - c.low_freq_factor) / (
                    c.high_freq_factor - c.low_freq_factor
                )
                blended = (1 - smooth) * f / c.scaling_factor + smooth * f
                scaled = torch.where(wavelen > lo_wl, f / c.scaling_factor, f)
                mid = (wavelen >= hi_wl) & (wavelen <= lo_wl)
                f = torch.where(mid, blended, scaled)
            elif c.scaling == "yarn" and c.max_seq_len > c.original_seq_len:
                def corr(rot):
                    return c.dim * math.log(c.original_seq_len / (rot * 2 * math.pi)) / (2 * math.log(c.theta))

                lo = max(math.floor(corr(c.beta_fast)), 0)
                hi = min(math.ceil(corr(c.beta_slow)), c.dim - 1)
                keep = 1 - _yarn_ramp(lo, hi, half)
                f = f / c.rope_factor * (1 - keep) + f * keep
            return f, 1.0
        # cos_sin flavour
        if c.scaling == "llama":
            raise NotImplementedError("Cos/sin RoPE does not support Llama scaling.")
        base = c.theta**expo
        if c.scaling == "yarn" and c.rope_factor > 1.0:
            mag = 0.1 * math.log(c.rope_factor) + 1.0
            d_half = c.dim / 2
            lo = d_half * math.log(c.original_seq_len / (c.beta_slow * 2 * math.pi)) / math.log(c.theta)
            hi = d_half * math.log(c.original_seq_len / (c.beta_fast * 2 * math.pi)) / math.log(c.theta)
            assert 0 < lo < hi < d_half - 1, f"Invalid YaRN params: 0 < {lo} < {hi} < {d_half - 1}"
            keep = 1 - ((torch.arange(half, dtype=torch.float32) - lo) / (hi - lo)).clamp(0, 1)
            f = (1.0 / (c.rope_factor * base)) * (1 - keep) + (1.0 / base) * keep
            return f, mag
        return 1.0 / base, 1.0

    def _precompute(self) -> torch.Tensor:
        f, mag = self.inv_freq()
        t = torch.arange(self.config.max_seq_len, device=f.device)
        ang = torch.outer(t, f).float()
        return torch.stack((ang.cos() * mag, ang.sin() * mag), dim=-1).contiguous()

    def forward(self, seq_len: int, positions: torch.Tensor | None = None) -> torch.Tensor:
        return self.cache

    def init_weights(self, **kwargs) -> None:
        dev = kwargs.get("buffer_device")
        if dev is not None:
            with torch.device(dev):
                self.cache = self._precompute()
        else:
            self.cache = self._precompute()


def apply_rotary_emb(xq, xk, table, positions=None, layout: str = "interleaved"):
    """Rotate query and key ``[B,S,H,Dh]`` with the (cos, sin) ``table``."""
    return ops.rope(xq, table, positions, layout), ops.rope(xk, table, positions, layout)


def apply_rotary_emb_single(x, table, positions=None, layout: str = "interleaved"):
    return ops.rope(x, table, positions, layout)
