"""Euler sampler of the rectified-flow ODE with the resolution-dependent time shift, classifier-free guidance, decoding
and PNG export. Parity: torchtitan/models/flux/inference/sampling.py."""

from __future__ import annotations

import math
import os

import torch

from ..utils import create_position_encoding_for_latents, generate_noise_latent, pack_latents, preprocess_data, unpack_latents


def time_shift(mu: float, sigma: float, t: torch.Tensor) -> torch.Tensor:
    return math.exp(mu) / (math.exp(mu) + (1 / t - 1) ** sigma)


def get_schedule(num_steps: int, image_seq_len: int, base_shift: float = 0.5, max_shift: float = 1.15, shift: bool = True) -> list[float]:
    ts = torch.linspace(1, 0, num_steps + 1)
    if shift:
        m = (max_shift - base_shift) / (4096 - 256)
        mu = m * image_seq_len + (base_shift - 256 * m)
        ts = time_shift(mu, 1.0, ts)
    return ts.tolist()


@torch.no_grad()
def denoise(model, latents, clip_enc, t5_enc, steps: int, cfg_scale: float = 1.0, empty_clip=None, empty_t5=None):
    bsz, _, lh, lw = latents.shape
    dev, dt = latents.device, latents.dtype
    img_ids = create_position_encoding_for_latents(bsz, lh, lw).to(dev)
    txt_ids = torch.zeros(bsz, t5_enc.shape[1], 3, device=dev)
    x = pack_latents(latents)
    ts = get_schedule(steps, x.shape[1])
    for t_cur, t_prev in zip(ts[:-1], ts[1:]):
        t_vec = torch.full((bsz,), t_cur, dtype=dt, device=dev)
        pred = model(img=x, img_ids=img_ids, txt=t5_enc, txt_ids=txt_ids, y=clip_enc, timesteps=t_vec)
        if cfg_scale != 1.0 and empty_clip is not None:
            un = model(img=x, img_ids=img_ids, txt=empty_t5, txt_ids=txt_ids, y=empty_clip, timesteps=t_vec)
            pred = un + cfg_scale * (pred - un)
        x = x + (t_prev - t_cur) * pred
    return unpack_latents(x, lh, lw)


@torch.no_grad()
def generate_image(device, dtype, *, model, autoencoder, clip_encoder, t5_encoder, clip_tokens, t5_tokens, height: int = 256,
                   width: int = 256, steps: int = 4, seed: int | None = 0, cfg_scale: float = 1.0) -> torch.Tensor:
    batch = preprocess_data(device, dtype, autoencoder=None, clip_encoder=clip_encoder, t5_encoder=t5_encoder,
                            batch={"clip_tokens": clip_tokens, "t5_tokens": t5_tokens})
    lat = generate_noise_latent(clip_tokens.shape[0], height, width, device, dtype, seed)
    lat = denoise(model, lat, batch["clip_encodings"], batch["t5_encodings"], steps, cfg_scale)
    return autoencoder.decode(lat)


def save_image(img_chw: torch.Tensor, folder: str, name: str) -> str:
    """Write one decoded image ([-1, 1] range) as PNG."""
    from PIL import Image

    os.makedirs(folder, exist_ok=True)
    x = ((img_chw.float().clamp(-1, 1) + 1) * 127.5).round().to(torch.uint8).permute(1, 2, 0).cpu().numpy()
    path = os.path.join(folder, name)
    Image.fromarray(x).save(path)
    return path
