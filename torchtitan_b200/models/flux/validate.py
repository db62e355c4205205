"""Validation for FLUX: flow-matching loss at fixed, evenly spaced timesteps on held-out batches, optionally sampling a few
images and saving them as PNG files (torchtitan/models/flux/validate.py)."""

from __future__ import annotations

import os

import torch

from .inference.sampling import generate_image, save_image
from .utils import create_position_encoding_for_latents, pack_latents, preprocess_data


class FluxValidator:
    def __init__(self, trainer, steps: int = 4, timesteps: int = 8, save_img_count: int = 0, save_img_folder: str = "img"):
        self.t, self.steps, self.n_t, self.save_img_count, self.save_img_folder = trainer, steps, timesteps, save_img_count, save_img_folder

    @torch.no_grad()
    def validate(self, data_iterator, step: int) -> float:
        tr = self.t
        model = tr.model_parts[0]
        model.eval()
        total, count = 0.0, 0
        for _ in range(self.steps):
            inputs, images = next(data_iterator)
            batch = preprocess_data(tr.device, tr._dtype, autoencoder=tr.autoencoder, clip_encoder=tr.clip_encoder,
                                    t5_encoder=tr.t5_encoder, batch={**inputs, "image": images})
            x = batch["img_encodings"]
            bsz, _, lh, lw = x.shape
            img_ids = create_position_encoding_for_latents(bsz, lh, lw).to(tr.device)
            txt_ids = torch.zeros(bsz, batch["t5_encodings"].shape[1], 3, device=tr.device)
            for k in range(self.n_t):
                t = torch.full((bsz,), (k + 0.5) / self.n_t, device=tr.device)
                noise = torch.randn_like(x)
                sig = t.view(-1, 1, 1, 1).to(x.dtype)
                pred = model(img=pack_latents((1 - sig) * x + sig * noise), img_ids=img_ids, txt=batch["t5_encodings"], txt_ids=txt_ids,
                             y=batch["clip_encodings"], timesteps=t.to(x.dtype))
                total += float(torch.nn.functional.mse_loss(pred.float(), pack_latents(noise - x).float()))
                count += 1
            if self.save_img_count:
                imgs = generate_image(tr.device, tr._dtype, model=model, autoencoder=tr.autoencoder, clip_encoder=tr.clip_encoder,
                                      t5_encoder=tr.t5_encoder, clip_tokens=inputs["clip_tokens"][: self.save_img_count],
                                      t5_tokens=inputs["t5_tokens"][: self.save_img_count], height=images.shape[-2], width=images.shape[-1])
                for i, im in enumerate(imgs):
                    save_image(im, os.path.join(tr.config.dump_folder, self.save_img_folder), f"step{step}_img{i}.png")
        model.train()
        return total / max(1, count)
