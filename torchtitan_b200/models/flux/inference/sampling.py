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
    """Euler steps from noise (t = 1) to the image latents (t = 0). With classifier-free guidance
    (``cfg_scale != 1`` and the encodings of the empty prompt given) the unconditional and the conditional branch run as
    one batch of twice the size and ``pred = uncond + scale * (cond - uncond)``
    (torchtitan/models/flux/inference/sampling.py:179-250)."""
    bsz, _, lh, lw = latents.shape
    dev, dt = latents.device, latents.dtype
    guided = cfg_scale != 1.0 and empty_clip is not None and empty_t5 is not None
    x = pack_latents(latents)
    if guided:
        t5_enc, clip_enc = torch.cat([empty_t5, t5_enc]), torch.cat([empty_clip, clip_enc])
    n = 2 * bsz if guided else bsz
    img_ids = create_position_encoding_for_latents(n, lh, lw).to(dev)
    txt_ids = torch.zeros(n, t5_enc.shape[1], 3, device=dev)
    ts = get_schedule(steps, x.shape[1])
    for t_cur, t_prev in zip(ts[:-1], ts[1:]):
        t_vec = torch.full((n,), t_cur, dtype=dt, device=dev)
        pred = model(img=torch.cat([x, x]) if guided else x, img_ids=img_ids, txt=t5_enc, txt_ids=txt_ids, y=clip_enc, timesteps=t_vec)
        if guided:
            un, co = pred.chunk(2)
            pred = un + cfg_scale * (co - un)
        x = x + (t_prev - t_cur) * pred
    return unpack_latents(x, lh, lw)


def _rows(tokens: torch.Tensor) -> torch.Tensor:
    return tokens if tokens.dim() == 2 else tokens.reshape(-1, tokens.shape[-1])


@torch.no_grad()
def generate_image(device, dtype, *, model, autoencoder, clip_encoder, t5_encoder, clip_tokens=None, t5_tokens=None,
                   prompt: str | list[str] | None = None, clip_tokenizer=None, t5_tokenizer=None, job_config=None,
                   height: int | None = None, width: int | None = None, steps: int | None = None, seed: int | None = 0,
                   cfg_scale: float | None = None) -> torch.Tensor:
    """Images [B, 3, H, W] in [-1, 1] for ``prompt`` (tokenised here) or for given token rows.

    ``job_config`` (a FLUX trainer configuration) supplies what is not passed: the resolution of the validation loader,
    ``validation.denoising_steps`` and the guidance switch and scale, as in the reference's ``generate_image``
    (sampling.py:72-176). Guidance needs the tokenizers (for the empty prompt)."""
    val = getattr(job_config, "validation", None)
    if steps is None:
        steps = val.denoising_steps if val is not None else 4
    if cfg_scale is None:
        cfg_scale = val.classifier_free_guidance_scale if val is not None and val.enable_classifier_free_guidance else 1.0
    if height is None or width is None:
        size = job_config.validator.dataloader.img_size if job_config is not None else 256
        height = width = 16 * (size // 16)
    if prompt is not None:
        prompt = [prompt] if isinstance(prompt, str) else list(prompt)
        clip_tokens, t5_tokens = clip_tokenizer.encode(prompt), t5_tokenizer.encode(prompt)
    clip_tokens, t5_tokens = _rows(clip_tokens), _rows(t5_tokens)
    n = clip_tokens.shape[0]
    batch = preprocess_data(device, dtype, autoencoder=None, clip_encoder=clip_encoder, t5_encoder=t5_encoder,
                            batch={"clip_tokens": clip_tokens, "t5_tokens": t5_tokens})
    empty = {"clip_encodings": None, "t5_encodings": None}
    if cfg_scale != 1.0:
        if clip_tokenizer is None or t5_tokenizer is None:
            raise ValueError("classifier-free guidance needs the two tokenizers to encode the empty prompt")
        empty = preprocess_data(device, dtype, autoencoder=None, clip_encoder=clip_encoder, t5_encoder=t5_encoder,
                                batch={"clip_tokens": _rows(clip_tokenizer.encode("")).repeat(n, 1),
                                       "t5_tokens": _rows(t5_tokenizer.encode("")).repeat(n, 1)})
    lat = generate_noise_latent(n, height, width, device, dtype, seed)
    lat = denoise(model, lat, batch["clip_encodings"], batch["t5_encodings"], steps, cfg_scale,
                  empty_clip=empty["clip_encodings"], empty_t5=empty["t5_encodings"])
    return autoencoder.decode(lat)


def save_image(img_chw: torch.Tensor, folder: str, name: str, prompt: str | None = None) -> str:
    """Write one decoded image ([-1, 1] range, [3, H, W] or [1, 3, H, W]) as PNG / JPEG. The file carries EXIF fields
    marking it as generated (software, model = file name) and, when given, the prompt as image description."""
    from PIL import ExifTags, Image

    os.makedirs(folder, exist_ok=True)
    if img_chw.dim() == 4:
        img_chw = img_chw[0]
    x = ((img_chw.float().clamp(-1, 1) + 1) * 127.5).round().to(torch.uint8).permute(1, 2, 0).cpu().numpy()
    path = os.path.join(folder, name)
    exif = Image.Exif()
    exif[ExifTags.Base.Software] = "AI generated;txt2img;flux"
    exif[ExifTags.Base.Model] = name
    if prompt is not None:
        exif[ExifTags.Base.ImageDescription] = prompt
    Image.fromarray(x).save(path, exif=exif)
    return path
