"""Latent packing, position ids and batch preprocessing for FLUX (torchtitan/models/flux/utils.py)."""

from __future__ import annotations

import torch
from torch import Tensor

PATCH = 2


def preprocess_data(device, dtype, *, autoencoder, clip_encoder, t5_encoder, batch: dict) -> dict:
    clip_tokens = batch["clip_tokens"].squeeze(1).to(device=device, dtype=torch.int)
    t5_tokens = batch["t5_tokens"].squeeze(1).to(device=device, dtype=torch.int)
    batch["clip_encodings"] = clip_encoder(clip_tokens).to(dtype)
    batch["t5_encodings"] = t5_encoder(t5_tokens).to(dtype)
    if autoencoder is not None:
        batch["img_encodings"] = autoencoder.encode(batch["image"].to(device=device, dtype=dtype)).to(device=device, dtype=dtype)
    return batch


def generate_noise_latent(bsz: int, height: int, width: int, device, dtype, seed: int | None = None) -> Tensor:
    g = None if seed is None else torch.Generator().manual_seed(seed)
    return torch.randn(bsz, 16, height // 8, width // 8, dtype=dtype, generator=g).to(device)


def create_position_encoding_for_latents(bsz: int, latent_height: int, latent_width: int, position_dim: int = 3) -> Tensor:
    h, w = latent_height // PATCH, latent_width // PATCH
    pos = torch.zeros(h, w, position_dim)
    pos[:, :, 1] = torch.arange(h).unsqueeze(1)
    pos[:, :, 2] = torch.arange(w).unsqueeze(0)
    return pos.view(1, h * w, position_dim).repeat(bsz, 1, 1)


def pack_latents(x: Tensor) -> Tensor:
    """[b, c, h*2, w*2] -> [b, h*w, c*4]"""
    b, c, H, W = x.shape
    h, w = H // PATCH, W // PATCH
    return x.reshape(b, c, h, PATCH, w, PATCH).permute(0, 2, 4, 1, 3, 5).reshape(b, h * w, c * PATCH * PATCH)


def unpack_latents(x: Tensor, latent_height: int, latent_width: int) -> Tensor:
    b, _, cpp = x.shape
    h, w, c = latent_height // PATCH, latent_width // PATCH, cpp // (PATCH * PATCH)
    return x.reshape(b, h, w, c, PATCH, PATCH).permute(0, 3, 1, 4, 2, 5).reshape(b, c, h * PATCH, w * PATCH)
