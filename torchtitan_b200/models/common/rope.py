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


# ------------------------------------------------------------------------------------ the reference's cache layouts
# The models of this framework keep one table layout ([max_seq_len, head_dim / 2, 2] = cos, sin) and rotate through
# ``ops.rope``. Code written against the reference passes its two cache layouts instead
# (torchtitan/models/common/rope.py:293-360); the functions below take those, compute in fp32 and return the input dtype.
def _rows_for(cache: torch.Tensor, x: torch.Tensor, positions: torch.Tensor | None) -> torch.Tensor:
    """Cache rows for every token of ``x`` [B, S, H, D], shaped to broadcast over heads: [1 | B, S, 1, ...]."""
    if positions is None:
        return cache[: x.shape[1]].unsqueeze(0).unsqueeze(2)
    rows = cache[positions.long()]                       # [1 | B, S, ...]
    return rows.unsqueeze(2)


def apply_rotary_emb_cos_sin(xq: torch.Tensor, xk: torch.Tensor, rope_cache: torch.Tensor, positions: torch.Tensor | None = None):
    """Half-rotation RoPE with a ``[max_seq_len, 2 * head_dim]`` cache holding cos and sin side by side, each over the
    whole head dimension (the two halves repeat)."""
    d = xq.shape[-1]
    tab = _rows_for(rope_cache, xq, positions).to(device=xq.device, dtype=torch.float32)
    cos, sin = tab[..., :d], tab[..., d:]

    def rotate(x):
        xf = x.float()
        half = torch.cat((-xf[..., d // 2:], xf[..., : d // 2]), dim=-1)
        return (xf * cos + half * sin).type_as(x)

    return rotate(xq), rotate(xk)


def apply_rotary_emb_single_complex(x: torch.Tensor, freqs_cis: torch.Tensor, positions: torch.Tensor | None = None):
    """Interleaved-pair RoPE with a complex ``[max_seq_len, head_dim / 2]`` cache (``exp(i * angle)``)."""
    rows = _rows_for(freqs_cis, x, positions).to(x.device)
    xc = torch.view_as_complex(x.float().reshape(*x.shape[:-1], -1, 2))
    return torch.view_as_real(xc * rows).flatten(-2).type_as(x)


def apply_rotary_emb_complex(xq: torch.Tensor, xk: torch.Tensor, freqs_cis: torch.Tensor, positions: torch.Tensor | None = None):
    return apply_rotary_emb_single_complex(xq, freqs_cis, positions), apply_rotary_emb_single_complex(xk, freqs_cis, positions)
