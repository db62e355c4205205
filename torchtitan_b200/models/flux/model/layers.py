"""FLUX.1 transformer layers: 3-axis rotary position embedding, timestep / vector embedders, adaptive-LayerNorm
modulation, double-stream (image and text streams with joint attention) and single-stream blocks, final layer.
Parity: torchtitan/models/flux/model/layers.py. Attention is bidirectional (non-causal) over the concatenated text +
image sequence and runs through ``ops.attention`` (head dim 128 -> the flash kernel on a GPU)."""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from torchtitan_b200 import ops
from torchtitan_b200.protocols.module import Module


def rope(pos: torch.Tensor, dim: int, theta: int) -> torch.Tensor:
    """[..., n] positions -> [..., n, dim/2, 2, 2] rotation matrices."""
    assert dim % 2 == 0
    scale = torch.arange(0, dim, 2, dtype=torch.float64, device=pos.device) / dim
    omega = 1.0 / (theta**scale)
    out = pos.double().unsqueeze(-1) * omega
    out = torch.stack((torch.cos(out), -torch.sin(out), torch.sin(out), torch.cos(out)), dim=-1)
    return out.reshape(*out.shape[:-1], 2, 2).float()


def apply_rope(xq, xk, freqs_cis):
    """xq/xk [B, H, L, D]; freqs_cis [B, 1, L, D/2, 2, 2]."""
    def rot(x):
        x_ = x.float().reshape(*x.shape[:-1], -1, 1, 2)
        out = freqs_cis[..., 0] * x_[..., 0] + freqs_cis[..., 1] * x_[..., 1]
        return out.reshape(*x.shape).type_as(x)

    return rot(xq), rot(xk)


class EmbedND(Module):
    def __init__(self, dim: int, theta: int, axes_dim: tuple[int, ...]):
        super().__init__()
        self.dim, self.theta, self.axes_dim = dim, theta, tuple(axes_dim)

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        emb = torch.cat([rope(ids[..., i], self.axes_dim[i], self.theta) for i in range(ids.shape[-1])], dim=-3)
        return emb.unsqueeze(1)

    def init_weights(self, **kwargs) -> None:
        return None


def timestep_embedding(t: torch.Tensor, dim: int, max_period: int = 10000, time_factor: float = 1000.0) -> torch.Tensor:
    t = time_factor * t
    half = dim // 2
    freqs = torch.exp(-math.log(max_period) * torch.arange(half, dtype=torch.float32, device=t.device) / half)
    args = t[:, None].float() * freqs[None]
    emb = torch.cat((torch.cos(args), torch.sin(args)), dim=-1)
    if dim % 2:
        emb = torch.cat((emb, torch.zeros_like(emb[:, :1])), dim=-1)
    return emb.to(t) if torch.is_floating_point(t) else emb


class MLPEmbedder(Module):
    def __init__(self, in_dim: int, hidden_dim: int):
        super().__init__()
        self.in_layer, self.out_layer = nn.Linear(in_dim, hidden_dim), nn.Linear(hidden_dim, hidden_dim)

    def forward(self, x):
        return self.out_layer(F.silu(self.in_layer(x)))

    def init_weights(self, init_std: float = 0.02, **kwargs) -> None:
        for m in (self.in_layer, self.out_layer):
            nn.init.normal_(m.weight, std=init_std)
            nn.init.zeros_(m.bias)


class QKNorm(Module):
    def __init__(self, dim: int):
        super().__init__()
        self.query_norm, self.key_norm = nn.RMSNorm(dim), nn.RMSNorm(dim)

    def forward(self, q, k, v):
        return self.query_norm(q).to(v), self.key_norm(k).to(v)

    def init_weights(self, **kwargs) -> None:
        self.query_norm.reset_parameters()
        self.key_norm.reset_parameters()


def _attend(q, k, v, pe):
    """q,k,v [B, H, L, D] -> [B, L, H*D]; full (non-causal) attention after rotary embedding."""
    q, k = apply_rope(q, k, pe)
    o = ops.attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), causal=False)
    return o.reshape(o.shape[0], o.shape[1], -1)


class SelfAttention(Module):
    def __init__(self, dim: int, num_heads: int = 8, qkv_bias: bool = False):
        super().__init__()
        self.num_heads = num_heads
        self.qkv = nn.Linear(dim, dim * 3, bias=qkv_bias)
        self.norm = QKNorm(dim // num_heads)
        self.proj = nn.Linear(dim, dim)

    def split(self, x):
        B, L, _ = x.shape
        qkv = self.qkv(x).view(B, L, 3, self.num_heads, -1).permute(2, 0, 3, 1, 4)
        q, k = self.norm(qkv[0], qkv[1], qkv[2])
        return q, k, qkv[2]

    def init_weights(self, **kwargs) -> None:
        for m in (self.qkv, self.proj):
            nn.init.xavier_uniform_(m.weight)
            if m.bias is not None:
                nn.init.zeros_(m.bias)
        self.norm.init_weights()


@dataclass
class ModulationOut:
    shift: torch.Tensor
    scale: torch.Tensor
    gate: torch.Tensor


class Modulation(Module):
    def __init__(self, dim: int, double: bool):
        super().__init__()
        self.is_double, self.multiplier = double, 6 if double else 3
        self.lin = nn.Linear(dim, self.multiplier * dim)

    def forward(self, vec):
        out = self.lin(F.silu(vec))[:, None, :].chunk(self.multiplier, dim=-1)
        return ModulationOut(*out[:3]), (ModulationOut(*out[3:]) if self.is_double else None)

    def init_weights(self, **kwargs) -> None:
        nn.init.zeros_(self.lin.weight)
        nn.init.zeros_(self.lin.bias)


def _mlp(dim: int, hidden: int) -> nn.Sequential:
    return nn.Sequential(nn.Linear(dim, hidden), nn.GELU(approximate="tanh"), nn.Linear(hidden, dim))


class DoubleStreamBlock(Module):
    def __init__(self, hidden_size: int, num_heads: int, mlp_ratio: float, qkv_bias: bool = False):
        super().__init__()
        hidden = int(hidden_size * mlp_ratio)
        self.num_heads = num_heads
        self.img_mod, self.txt_mod = Modulation(hidden_size, True), Modulation(hidden_size, True)
        self.img_norm1, self.txt_norm1, self.img_norm2, self.txt_norm2 = (
            nn.LayerNorm(hidden_size, elementwise_affine=False, eps=1e-6) for _ in range(4))
        self.img_attn, self.txt_attn = SelfAttention(hidden_size, num_heads, qkv_bias), SelfAttention(hidden_size, num_heads, qkv_bias)
        self.img_mlp, self.txt_mlp = _mlp(hidden_size, hidden), _mlp(hidden_size, hidden)

    def forward(self, img, txt, vec, pe):
        im1, im2 = self.img_mod(vec)
        tm1, tm2 = self.txt_mod(vec)
        iq, ik, iv = self.img_attn.split((1 + im1.scale) * self.img_norm1(img) + im1.shift)
        tq, tk, tv = self.txt_attn.split((1 + tm1.scale) * self.txt_norm1(txt) + tm1.shift)
        attn = _attend(torch.cat((tq, iq), 2), torch.cat((tk, ik), 2), torch.cat((tv, iv), 2), pe)
        t_attn, i_attn = attn[:, : txt.shape[1]], attn[:, txt.shape[1] :]
        img = img + im1.gate * self.img_attn.proj(i_attn)
        img = img + im2.gate * self.img_mlp((1 + im2.scale) * self.img_norm2(img) + im2.shift)
        txt = txt + tm1.gate * self.txt_attn.proj(t_attn)
        txt = txt + tm2.gate * self.txt_mlp((1 + tm2.scale) * self.txt_norm2(txt) + tm2.shift)
        return img, txt

    def init_weights(self, **kwargs) -> None:
        for m in (self.img_mod, self.txt_mod, self.img_attn, self.txt_attn):
            m.init_weights()
        for mlp in (self.img_mlp, self.txt_mlp):
            for m in (mlp[0], mlp[2]):
                nn.init.xavier_uniform_(m.weight)
                nn.init.zeros_(m.bias)


class SingleStreamBlock(Module):
    def __init__(self, hidden_size: int, num_heads: int, mlp_ratio: float = 4.0):
        super().__init__()
        self.hidden_dim, self.num_heads = hidden_size, num_heads
        self.mlp_hidden_dim = int(hidden_size * mlp_ratio)
        self.linear1 = nn.Linear(hidden_size, hidden_size * 3 + self.mlp_hidden_dim)
        self.linear2 = nn.Linear(hidden_size + self.mlp_hidden_dim, hidden_size)
        self.norm = QKNorm(hidden_size // num_heads)
        self.pre_norm = nn.LayerNorm(hidden_size, elementwise_affine=False, eps=1e-6)
        self.modulation = Modulation(hidden_size, False)

    def forward(self, x, vec, pe):
        mod, _ = self.modulation(vec)
        qkv, mlp = torch.split(self.linear1((1 + mod.scale) * self.pre_norm(x) + mod.shift), [3 * self.hidden_dim, self.mlp_hidden_dim], dim=-1)
        B, L, _ = qkv.shape
        qkv = qkv.view(B, L, 3, self.num_heads, -1).permute(2, 0, 3, 1, 4)
        q, k = self.norm(qkv[0], qkv[1], qkv[2])
        attn = _attend(q, k, qkv[2], pe)
        return x + mod.gate * self.linear2(torch.cat((attn, F.gelu(mlp, approximate="tanh")), 2))

    def init_weights(self, **kwargs) -> None:
        for m in (self.linear1, self.linear2):
            nn.init.xavier_uniform_(m.weight)
            nn.init.zeros_(m.bias)
        self.norm.init_weights()
        self.modulation.init_weights()


class LastLayer(Module):
    def __init__(self, hidden_size: int, patch_size: int, out_channels: int):
        super().__init__()
        self.norm_final = nn.LayerNorm(hidden_size, elementwise_affine=False, eps=1e-6)
        self.linear = nn.Linear(hidden_size, patch_size * patch_size * out_channels)
        self.adaLN_modulation = nn.Sequential(nn.SiLU(), nn.Linear(hidden_size, 2 * hidden_size))

    def forward(self, x, vec):
        shift, scale = self.adaLN_modulation(vec).chunk(2, dim=1)
        return self.linear((1 + scale[:, None, :]) * self.norm_final(x) + shift[:, None, :])

    def init_weights(self, **kwargs) -> None:
        for m in (self.adaLN_modulation[-1], self.linear):
            nn.init.zeros_(m.weight)
            nn.init.zeros_(m.bias)
