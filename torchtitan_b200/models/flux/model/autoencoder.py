"""The FLUX latent autoencoder (convolutional encoder / decoder with a diagonal Gaussian bottleneck); frozen during
training. Parity: torchtitan/models/flux/model/autoencoder.py."""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class AutoEncoderParams:
    resolution: int = 256
    in_channels: int = 3
    ch: int = 128
    out_ch: int = 3
    ch_mult: tuple = (1, 2, 4, 4)
    num_res_blocks: int = 2
    z_channels: int = 16
    scale_factor: float = 0.3611
    shift_factor: float = 0.1159


def _norm(c: int) -> nn.GroupNorm:
    return nn.GroupNorm(num_groups=min(32, c), num_channels=c, eps=1e-6, affine=True)


class AttnBlock(nn.Module):
    def __init__(self, c: int):
        super().__init__()
        self.norm = _norm(c)
        self.q, self.k, self.v, self.proj_out = (nn.Conv2d(c, c, 1) for _ in range(4))

    def forward(self, x):
        h = self.norm(x)
        B, C, H, W = h.shape
        q, k, v = (m(h).reshape(B, 1, C, H * W).transpose(2, 3) for m in (self.q, self.k, self.v))
        o = F.scaled_dot_product_attention(q, k, v).transpose(2, 3).reshape(B, C, H, W)
        return x + self.proj_out(o)


class ResnetBlock(nn.Module):
    def __init__(self, cin: int, cout: int):
        super().__init__()
        self.norm1, self.conv1 = _norm(cin), nn.Conv2d(cin, cout, 3, padding=1)
        self.norm2, self.conv2 = _norm(cout), nn.Conv2d(cout, cout, 3, padding=1)
        self.nin_shortcut = nn.Conv2d(cin, cout, 1) if cin != cout else None

    def forward(self, x):
        h = self.conv1(F.silu(self.norm1(x)))
        h = self.conv2(F.silu(self.norm2(h)))
        return (x if self.nin_shortcut is None else self.nin_shortcut(x)) + h


class Encoder(nn.Module):
    def __init__(self, p: AutoEncoderParams):
        super().__init__()
        self.conv_in = nn.Conv2d(p.in_channels, p.ch, 3, padding=1)
        chans = [p.ch * m for m in (1,) + tuple(p.ch_mult)]
        self.down = nn.ModuleList()
        for i in range(len(p.ch_mult)):
            blocks = nn.ModuleList(ResnetBlock(chans[i] if j == 0 else chans[i + 1], chans[i + 1]) for j in range(p.num_res_blocks))
            level = nn.Module()
            level.block = blocks
            level.downsample = nn.Conv2d(chans[i + 1], chans[i + 1], 3, stride=2, padding=0) if i != len(p.ch_mult) - 1 else None
            self.down.append(level)
        c = chans[-1]
        self.mid_block_1, self.mid_attn_1, self.mid_block_2 = ResnetBlock(c, c), AttnBlock(c), ResnetBlock(c, c)
        self.norm_out, self.conv_out = _norm(c), nn.Conv2d(c, 2 * p.z_channels, 3, padding=1)

    def forward(self, x):
        h = self.conv_in(x)
        for level in self.down:
            for b in level.block:
                h = b(h)
            if level.downsample is not None:
                h = level.downsample(F.pad(h, (0, 1, 0, 1)))
        h = self.mid_block_2(self.mid_attn_1(self.mid_block_1(h)))
        return self.conv_out(F.silu(self.norm_out(h)))


class Decoder(nn.Module):
    def __init__(self, p: AutoEncoderParams):
        super().__init__()
        c = p.ch * p.ch_mult[-1]
        self.conv_in = nn.Conv2d(p.z_channels, c, 3, padding=1)
        self.mid_block_1, self.mid_attn_1, self.mid_block_2 = ResnetBlock(c, c), AttnBlock(c), ResnetBlock(c, c)
        self.up = nn.ModuleList()
        for i in reversed(range(len(p.ch_mult))):
            cout = p.ch * p.ch_mult[i]
            level = nn.Module()
            level.block = nn.ModuleList(ResnetBlock(c if j == 0 else cout, cout) for j in range(p.num_res_blocks + 1))
            level.upsample = nn.Conv2d(cout, cout, 3, padding=1) if i != 0 else None
            c = cout
            self.up.append(level)
        self.norm_out, self.conv_out = _norm(c), nn.Conv2d(c, p.out_ch, 3, padding=1)

    def forward(self, z):
        h = self.mid_block_2(self.mid_attn_1(self.mid_block_1(self.conv_in(z))))
        for level in self.up:
            for b in level.block:
                h = b(h)
            if level.upsample is not None:
                h = level.upsample(F.interpolate(h, scale_factor=2.0, mode="nearest"))
        return self.conv_out(F.silu(self.norm_out(h)))


class AutoEncoder(nn.Module):
    def __init__(self, params: AutoEncoderParams):
        super().__init__()
        self.params = params
        self.encoder, self.decoder = Encoder(params), Decoder(params)

    def encode(self, x: torch.Tensor, sample: bool = True) -> torch.Tensor:
        mean, logvar = torch.chunk(self.encoder(x), 2, dim=1)
        z = mean + torch.exp(0.5 * logvar) * torch.randn_like(mean) if sample else mean
        return self.params.scale_factor * (z - self.params.shift_factor)

    def decode(self, z: torch.Tensor) -> torch.Tensor:
        return self.decoder(z / self.params.scale_factor + self.params.shift_factor)

    def forward(self, x):
        return self.decode(self.encode(x))


def load_ae(ckpt_path: str, params: AutoEncoderParams, device="cpu", dtype=torch.bfloat16, random_init: bool = False) -> AutoEncoder:
    ae = AutoEncoder(params)
    if not random_init:
        import os

        if not os.path.exists(ckpt_path):
            raise ValueError(f"Autoencoder path {ckpt_path} does not exist. Please download it first.")
        from safetensors.torch import load_file

        ae.load_state_dict(load_file(ckpt_path), strict=False)
    return ae.to(device=device, dtype=dtype).requires_grad_(False)
